// Small kernels of the cache's append path.
//   rope        : rotary embedding of new K tokens, op for op like the reference's
//                 apply_rotary_pos_emb_single (utils/compute.py:22-43): (t*cos) + (rotate_half(t)*sin),
//                 each op rounded to the element type.
//   append      : rope (optional) on the new K tokens + copy of the new V tokens into the residual
//                 buffers, one launch per decode step and layer.
//   dequantize  : codes + scale/zero -> dense K or V exactly as the reference's cache does it,
//                 (code + zero) * scale or code * scale + min (utils/compute.py:173-178); used when a
//                 caller asks for the dense history (prefill attention, debugging).
#include "common.cuh"
#include "launch.h"

namespace pkv {

template <typename T> struct CT;
template <> struct CT<__half> {
    static __device__ __forceinline__ float ld(const __half* p) { return __half2float(*p); }
    static __device__ __forceinline__ float rnd(float x) { return __half2float(__float2half_rn(x)); }
    static __device__ __forceinline__ __half cvt(float x) { return __float2half_rn(x); }
};
template <> struct CT<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ float rnd(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
    static __device__ __forceinline__ __nv_bfloat16 cvt(float x) { return __float2bfloat16_rn(x); }
};

// grid (tokens, heads, batch), 128 threads = channels
template <typename T>
__global__ void __launch_bounds__(128) rope_kernel(RopeArgs r) {
    const int t = blockIdx.x, h = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
    if (d >= r.dim) return;
    const T* x = reinterpret_cast<const T*>(r.x) + (int64_t)b * r.x_stride_b + (int64_t)h * r.x_stride_h + (int64_t)t * r.x_stride_s;
    const T* cs = reinterpret_cast<const T*>(r.cos) + (int64_t)b * r.cs_stride_b + (int64_t)t * r.dim;
    const T* sn = reinterpret_cast<const T*>(r.sin) + (int64_t)b * r.cs_stride_b + (int64_t)t * r.dim;
    const int half = r.dim / 2;
    const float v = CT<T>::ld(x + d);
    const float rot = d < half ? -CT<T>::ld(x + d + half) : CT<T>::ld(x + d - half);
    const float a = CT<T>::rnd(v * CT<T>::ld(cs + d));
    const float c = CT<T>::rnd(rot * CT<T>::ld(sn + d));
    T* o = reinterpret_cast<T*>(r.out) + (int64_t)b * r.o_stride_b + (int64_t)h * r.o_stride_h + (int64_t)t * r.o_stride_s;
    o[d] = CT<T>::cvt(a + c);
}

// Append of new tokens to the uncompressed residual in one launch: K is rotated (or copied when the
// caller already applied RoPE: cos == nullptr) and V copied to rows [position, position + tokens).
// grid (tokens, heads, batch), 128 threads = channels
template <typename T>
__global__ void __launch_bounds__(128) append_kernel(AppendArgs r) {
    const int t = blockIdx.x, h = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
    const T* x = reinterpret_cast<const T*>(r.k) + (int64_t)b * r.k_stride_b + (int64_t)h * r.k_stride_h + (int64_t)t * r.k_stride_s;
    const T* y = reinterpret_cast<const T*>(r.v) + (int64_t)b * r.v_stride_b + (int64_t)h * r.v_stride_h + (int64_t)t * r.v_stride_s;
    const int64_t o = (int64_t)b * r.res_stride_b + (int64_t)h * r.res_stride_h + (int64_t)(r.position + t) * 128 + d;
    T kv = x[d];
    if (r.cos) {
        const T* cs = reinterpret_cast<const T*>(r.cos) + (int64_t)b * r.cs_stride_b + (int64_t)t * 128;
        const T* sn = reinterpret_cast<const T*>(r.sin) + (int64_t)b * r.cs_stride_b + (int64_t)t * 128;
        const float rot = d < 64 ? -CT<T>::ld(x + d + 64) : CT<T>::ld(x + d - 64);
        const float a = CT<T>::rnd(CT<T>::ld(x + d) * CT<T>::ld(cs + d));
        const float c = CT<T>::rnd(rot * CT<T>::ld(sn + d));
        kv = CT<T>::cvt(a + c);
    }
    reinterpret_cast<T*>(r.k_res)[o] = kv;
    reinterpret_cast<T*>(r.v_res)[o] = y[d];
}

// grid (tokens, heads, batch), 128 threads = channels
template <typename T, bool HP>
__global__ void __launch_bounds__(128) dequant_kernel(DequantArgs q) {
    const int t = blockIdx.x, h = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
    const float code = (float)q.codes[(int64_t)b * q.codes_seq_stride + (int64_t)t * (q.heads * 128) + h * 128 + d];
    int64_t pi;
    if (q.mode == 0) pi = (((int64_t)b * q.heads + h) * q.param_blocks + (q.first_token + t) / q.block) * 128 + d;
    else if (q.mode == 1) pi = (int64_t)b * q.param_tokens + q.first_token + t;
    else if (q.mode == 2) pi = ((int64_t)b * q.heads + h) * q.param_tokens + q.first_token + t;      // vector: per (head, token)
    else pi = (int64_t)b * q.param_blocks + (q.first_token + t) / q.block;                           // block: per token block
    const float s = CT<T>::ld(reinterpret_cast<const T*>(q.scale) + pi), z = CT<T>::ld(reinterpret_cast<const T*>(q.zero) + pi);
    const float v = HP ? CT<T>::rnd(CT<T>::rnd(code * s) + z) : CT<T>::rnd(CT<T>::rnd(code + z) * s);
    reinterpret_cast<T*>(q.out)[(int64_t)b * q.o_stride_b + (int64_t)h * q.o_stride_h + (int64_t)t * q.o_stride_s + d] = CT<T>::cvt(v);
}

int launch_rope(const RopeArgs& r, cudaStream_t st) {
    if (r.batch < 0 || r.heads <= 0 || r.tokens < 0 || r.dim <= 0 || r.dim > 128 || (r.dim & 1)) return kBadArgument;
    if ((int64_t)r.batch * r.tokens == 0) return kOk;
    if (!r.x || !r.cos || !r.sin || !r.out) return kBadArgument;
    dim3 grid(r.tokens, r.heads, r.batch);
    if (r.is_bf16) rope_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(r);
    else rope_kernel<__half><<<grid, 128, 0, st>>>(r);
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

int launch_append(const AppendArgs& r, cudaStream_t st) {
    if (r.batch < 0 || r.heads <= 0 || r.tokens < 0 || r.position < 0 || r.position + r.tokens > r.res_capacity) return kBadArgument;
    if ((int64_t)r.batch * r.tokens == 0) return kOk;
    if (!r.k || !r.v || !r.k_res || !r.v_res || ((r.cos == nullptr) != (r.sin == nullptr))) return kBadArgument;
    dim3 grid(r.tokens, r.heads, r.batch);
    if (r.is_bf16) append_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(r);
    else append_kernel<__half><<<grid, 128, 0, st>>>(r);
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

int launch_dequantize(const DequantArgs& q, cudaStream_t st) {
    if (q.batch < 0 || q.heads <= 0 || q.tokens < 0 || q.block <= 0) return kBadArgument;
    if (q.mode < 0 || q.mode > 3) return kUnsupported;
    if ((int64_t)q.batch * q.tokens == 0) return kOk;
    if (!q.codes || !q.scale || !q.zero || !q.out) return kBadArgument;
    dim3 grid(q.tokens, q.heads, q.batch);
    if (q.is_bf16) { if (q.high_precision_zero) dequant_kernel<__nv_bfloat16, true><<<grid, 128, 0, st>>>(q); else dequant_kernel<__nv_bfloat16, false><<<grid, 128, 0, st>>>(q); }
    else           { if (q.high_precision_zero) dequant_kernel<__half, true><<<grid, 128, 0, st>>>(q); else dequant_kernel<__half, false><<<grid, 128, 0, st>>>(q); }
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

}  // namespace pkv
