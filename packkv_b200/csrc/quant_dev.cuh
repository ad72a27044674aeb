// The reference quantiser's arithmetic (utils/compute.py:84-112) as device code: every op in
// fp32, rounded back to the element type, round() = round-half-to-even.  Shared by quant.cu and
// fused_encode.cu.
#pragma once
#include "common.cuh"

namespace pkv {

template <typename T> struct QT;
template <> struct QT<__half> {
    static __device__ __forceinline__ float ld(const __half* p) { return __half2float(*p); }
    static __device__ __forceinline__ float rnd(float x) { return __half2float(__float2half_rn(x)); }
    static __device__ __forceinline__ __half cvt(float x) { return __float2half_rn(x); }
    // round(x rounded to the element type), as an integer: two conversions
    static __device__ __forceinline__ int rnd_to_int(float x) { return __half2int_rn(__float2half_rn(x)); }
    using T2 = __half2;
    static __device__ __forceinline__ T2 min2(T2 a, T2 b) { return __hmin2(a, b); }
    static __device__ __forceinline__ T2 max2(T2 a, T2 b) { return __hmax2(a, b); }
    static __device__ __forceinline__ T2 init2(float v) { return __float2half2_rn(v); }
    static __device__ __forceinline__ float lo_f(T2 a) { return __low2float(a); }
    static __device__ __forceinline__ float hi_f(T2 a) { return __high2float(a); }
    // Packed round-to-integer: adding 1536 to a value in [-512, 512) leaves a result in [1024, 2048),
    // where one ulp is 1, so the addition itself rounds half to even and the integer sits in the low
    // mantissa bits: bits = 0x6600 + round(q).
    static constexpr unsigned kIntBits = 0x6600u;
    static constexpr float kIntZeroLimit = 480.f;        // |zero| + 16 must stay below 512
    static constexpr float kHalfScaleMin = 0.0009765625f, kHalfScaleMax = 64.f, kHalfXMax = 500.f;   // 2^-10 .. 2^6, |x| * 128 finite
    static constexpr float kPre = 128.f;                 // residual computed on 128 x and 128 scale: stays out of the subnormals
    static __device__ __forceinline__ T2 dup(float v) { return __float2half2_rn(v); }
    static __device__ __forceinline__ T2 pair(float a, float b) { return __floats2half2_rn(a, b); }
    static __device__ __forceinline__ float2 to_float2(unsigned v) { return __half22float2(*reinterpret_cast<const __half2*>(&v)); }
    static __device__ __forceinline__ unsigned round2_bits(float a, float b) {
        const __half2 m = __hadd2(__floats2half2_rn(a, b), __float2half2_rn(1536.f));
        return *reinterpret_cast<const unsigned*>(&m);
    }
};
template <> struct QT<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ float rnd(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
    static __device__ __forceinline__ __nv_bfloat16 cvt(float x) { return __float2bfloat16_rn(x); }
    static __device__ __forceinline__ int rnd_to_int(float x) { return __bfloat162int_rn(__float2bfloat16_rn(x)); }
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ T2 min2(T2 a, T2 b) { return __hmin2(a, b); }
    static __device__ __forceinline__ T2 max2(T2 a, T2 b) { return __hmax2(a, b); }
    static __device__ __forceinline__ T2 init2(float v) { return __float2bfloat162_rn(v); }
    static __device__ __forceinline__ float lo_f(T2 a) { return __low2float(a); }
    static __device__ __forceinline__ float hi_f(T2 a) { return __high2float(a); }
    // as above with 192 and [-64, 64): bits = 0x4340 + round(q)
    static constexpr unsigned kIntBits = 0x4340u;
    static constexpr float kIntZeroLimit = 40.f;
    static constexpr float kHalfScaleMin = 7.450580596923828e-09f, kHalfScaleMax = 8192.f, kHalfXMax = 3.0e38f;   // 2^-27 .. 2^13
    static constexpr float kPre = 1.f;                   // bfloat16 has the exponent range of fp32: no prescale needed
    static __device__ __forceinline__ T2 dup(float v) { return __float2bfloat162_rn(v); }
    static __device__ __forceinline__ T2 pair(float a, float b) { return __floats2bfloat162_rn(a, b); }
    static __device__ __forceinline__ float2 to_float2(unsigned v) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v)); }
    static __device__ __forceinline__ unsigned round2_bits(float a, float b) {
        const __nv_bfloat162 m = __hadd2(__floats2bfloat162_rn(a, b), __float2bfloat162_rn(192.f));
        return *reinterpret_cast<const unsigned*>(&m);
    }
};

__device__ __forceinline__ unsigned min_u16x2(unsigned a, unsigned b) {
    unsigned d;
    asm("min.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ unsigned max_u16x2(unsigned a, unsigned b) {
    unsigned d;
    asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Quotient x / scale as PyTorch's half/bfloat16 kernels produce it (fp32 division, then rounding
// to the element type) at a fraction of the cost of an IEEE division per element: with the
// correctly rounded reciprocal r = RN(1/scale), q0 = x*r, e = fma(-scale, q0, x), q1 = fma(e, r, q0)
// is within one fp32 ulp of the exact quotient and exact whenever the quotient is representable.
// x and scale carry at most 11 significant bits, so the exact quotient is either exactly a rounding
// boundary of the element type (then q1 is exact) or at least one fp32 ulp away from every boundary:
// rounding q1 to the element type gives the same value as rounding the IEEE quotient.  Scales
// outside [1e-30, 1e30] (where r or the residual could leave the normal range) take the IEEE path.
template <typename T, bool HP>
struct Quantiser {
    float scale, zero, rcp;
    bool fast;
    __device__ __forceinline__ Quantiser() {}
    float xmax;          // largest |x| the parameters were derived from
    __device__ __forceinline__ Quantiser(float lo, float hi, float rel) {
        scale = QT<T>::rnd(QT<T>::rnd(hi - lo) * rel);
        zero = HP ? lo : QT<T>::rnd(rintf(QT<T>::rnd(__fdiv_rn(lo, scale))));
        xmax = fmaxf(fabsf(lo), fabsf(hi));
        prepare();
    }
    __device__ __forceinline__ void prepare() {
        const float m = fabsf(scale);
        fast = m > 1e-30f && m < 1e30f;
        rcp = __frcp_rn(scale);
    }
    template <bool FAST>
    __device__ __forceinline__ float quotient_t(float x) const {
        if (FAST) {
            const float q0 = x * rcp;
            return fmaf(fmaf(-scale, q0, x), rcp, q0);
        }
        return __fdiv_rn(x, scale);
    }
    // The code as a float.  round() of an element-type value is exact, and the final subtraction
    // of two small integers is exact whenever the code is in range, so those two roundings of the
    // reference are no-ops and are skipped; out-of-range codes are flagged by the caller.
    // FAST must only be true when `fast` is (callers decide once per warp, not per element).
    template <bool FAST>
    __device__ __forceinline__ float code_t(float x) const {
        if (HP) return rintf(QT<T>::rnd(quotient_t<FAST>(QT<T>::rnd(x - zero))));
        return rintf(QT<T>::rnd(quotient_t<FAST>(x))) - zero;
    }
    __device__ __forceinline__ float code(float x) const { return fast ? code_t<true>(x) : code_t<false>(x); }
    // The same code as an unsigned byte, saturated to 255 (negative, huge or NaN-derived values
    // all end at >= 2^bits... 255, which the callers' range check reports).  zero_i = (int)zero.
    template <bool FAST>
    __device__ __forceinline__ unsigned code_u8(float x, int zero_i) const {
        const int q = HP ? QT<T>::rnd_to_int(quotient_t<FAST>(QT<T>::rnd(x - zero))) : QT<T>::rnd_to_int(quotient_t<FAST>(x)) - zero_i;
        return min((unsigned)q, 255u);
    }
    // the packed two-element path needs the fast quotient and a zero-point small enough for the
    // packed round-to-integer (QT<T>::round2_bits)
    __device__ __forceinline__ bool packable() const { return fast && fabsf(zero) <= QT<T>::kIntZeroLimit; }
    // the quotient can be formed in the element type itself (HalfQuotient below): scale and |x| inside
    // the domain on which that arithmetic was checked exhaustively against the rounded IEEE quotient
    __device__ __forceinline__ bool half_domain() const {
        return packable() && scale >= QT<T>::kHalfScaleMin && scale <= QT<T>::kHalfScaleMax && xmax < QT<T>::kHalfXMax;
    }
    // parameters that cannot produce valid codes (constant channel: scale 0, or NaN / inf input)
    __device__ __forceinline__ bool degenerate() const { return !(scale > 0.f) || !(fabsf(zero) < 3.0e4f) || !(scale < 3.0e38f); }
};

// Codes of two elements (the two halves of `pair`, quantised by qa and qb) as two 16-bit lanes;
// kab = packed_code_bias(qa, qb).  Requires qa.packable() && qb.packable().
template <typename T>
__device__ __forceinline__ unsigned packed_code_bias(const Quantiser<T, false>& qa, const Quantiser<T, false>& qb) {
    return (QT<T>::kIntBits + (unsigned)(int)qa.zero) | ((QT<T>::kIntBits + (unsigned)(int)qb.zero) << 16);
}
template <typename T>
__device__ __forceinline__ unsigned packed_codes(unsigned pair, const Quantiser<T, false>& qa, const Quantiser<T, false>& qb, unsigned kab) {
    const float2 f = QT<T>::to_float2(pair);
    return QT<T>::round2_bits(qa.template quotient_t<true>(f.x), qb.template quotient_t<true>(f.y)) - kab;
}

// Quotient and integer code of two elements entirely in the element type (two elements per
// instruction, no conversion to fp32): r = RN(1/scale), q0 = x*r, e = fma(-scale, q0, x),
// q1 = fma(e, r, q0), then the packed round-to-integer.  For fp16 the residual is formed on
// 128*x and 128*scale (exact scalings) and multiplied by r/128, which keeps it out of the
// subnormal range where it would lose bits.  Checked exhaustively on the CPU (every scale in the
// half_domain() range x every x with |x/scale| <= 512, round-to-nearest-even arithmetic restated in
// double): round(q1) equals round(RN(x/scale)) for every pair, fp16 and bfloat16.
template <typename T>
struct HalfQuotient {
    typename QT<T>::T2 r, nsp, rp, magic, pre;
    unsigned kab;
    __device__ __forceinline__ HalfQuotient() {}
    __device__ __forceinline__ HalfQuotient(const Quantiser<T, false>& qa, const Quantiser<T, false>& qb) {
        const float ra = QT<T>::rnd(qa.rcp), rb = QT<T>::rnd(qb.rcp);
        r = QT<T>::pair(ra, rb);
        nsp = QT<T>::pair(-qa.scale * QT<T>::kPre, -qb.scale * QT<T>::kPre);
        rp = QT<T>::pair(ra / QT<T>::kPre, rb / QT<T>::kPre);
        magic = QT<T>::dup((float)(QT<T>::kIntBits == 0x6600u ? 1536 : 192));
        pre = QT<T>::dup(QT<T>::kPre);
        kab = packed_code_bias(qa, qb);
    }
    __device__ __forceinline__ unsigned codes(unsigned pair_bits) const {
        using T2 = typename QT<T>::T2;
        const T2 x = *reinterpret_cast<const T2*>(&pair_bits);
        const T2 xp = QT<T>::kPre == 1.f ? x : __hmul2(x, pre);
        const T2 q0 = __hmul2(x, r);
        const T2 e = __hfma2(nsp, q0, xp);
        const T2 m = __hadd2(__hfma2(e, rp, q0), magic);
        return *reinterpret_cast<const unsigned*>(&m) - kab;
    }
};

__device__ __forceinline__ unsigned code_byte(float c, float limit, bool& bad) {
    if (!(c >= 0.f && c < limit)) { bad = true; return 0u; }
    return (unsigned)c;
}

}  // namespace pkv
