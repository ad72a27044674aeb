// Shared device helpers for the PackKV sm_100a kernels: format constants, header bit
// fields, warp scans, unaligned byte-window loads.
//
// Stream format (byte-identical to the reference's CPU codec,
// packkv_cuda_ext/src/{k,v}_encode_cpu.cpp): a pack is 16 consecutive tokens of one channel,
// stored as min (RAW bits), len = bit_length(max-min) (LB bits) and a word
// W = sum_i (code_i - min) << (len*(15-i)) of 2*len bytes.  Header fields of the 32 lanes
// form a little-endian bit string, lane l at bit l*PPT*fbits, field i at +i*fbits.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

namespace pkv {

constexpr int kPackTokens = 16;
constexpr int kLanes = 32;

// status codes returned by the C ABI and OR-ed bit flags written to the device status word
enum Status : int {
    kOk = 0,
    kBadArgument = 1,
    kUnsupported = 2,
    kCudaError = 3,
};
enum DevFlag : unsigned {
    kFlagStreamOverflow = 1u,   // a block did not fit the stream capacity and was skipped
    kFlagCodeRange = 2u,        // a quantised code did not fit the requested bit width
    kFlagBadStream = 4u,        // a block_info entry or header points outside the stream
    kFlagTimeout = 8u,          // a bounded wait gave up
    kFlagZeroRange = 16u,       // a zero-point outside the range in which the in-kernel dequantisation is exact
};

__host__ __device__ constexpr int len_field_bits(int raw_bits) {
    // bits needed to store len in [0, raw_bits]: 4->3, 3->2, 2->2
    return raw_bits >= 4 ? 3 : 2;
}

// ---- geometry -------------------------------------------------------------------------
struct KGeom {
    int rounds;      // 16-token rounds per block
    int min_bytes;   // per round
    int len_bytes;   // per round
    int head_bytes;  // u16 round_end[rounds]
    __host__ __device__ KGeom(int cb, int bits)
        : rounds(cb / kPackTokens), min_bytes(bits * 16), len_bytes(len_field_bits(bits) * 16),
          head_bytes(2 * (cb / kPackTokens)) {}
};

struct VGeom {
    int rpw;         // segments per warp-half (64-token halves of a 128-token block)
    int ppt;         // packs per lane per segment
    int nseg;        // 2 * rpw
    int min_bytes;   // per segment
    int len_bytes;   // per segment
    int head_bytes;  // u16 seg_end[nseg]
    __host__ __device__ VGeom(int cb, int bits) {
        rpw = cb == 128 ? 2 : 1;
        ppt = cb == 32 ? 2 : 4;
        nseg = 2 * rpw;
        min_bytes = bits * ppt * 4;
        len_bytes = len_field_bits(bits) * ppt * 4;
        head_bytes = 2 * nseg;
    }
};

// ---- small bit helpers ----------------------------------------------------------------
__device__ __forceinline__ int bit_length_u32(unsigned v) { return 32 - __clz(v); }

__device__ __forceinline__ unsigned lane_id() { return threadIdx.x & 31u; }

// inclusive warp scan (add)
__device__ __forceinline__ unsigned warp_inclusive_sum(unsigned v) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        // the shuffle's own predicate says whether the source lane exists: no lane compare needed
        asm volatile("{ .reg .pred p; .reg .b32 n; shfl.sync.up.b32 n|p, %0, %1, 0, 0xffffffff; @p add.u32 %0, %0, n; }" : "+r"(v) : "r"(d));
    }
    return v;
}

__device__ __forceinline__ unsigned warp_sum(unsigned v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// Reads the lane word of `width` bits (<= 16) at bit lane*width of a byte string.
// Works for any byte pointer (shared or global), any alignment.
__device__ __forceinline__ unsigned load_lane_field(const uint8_t* hdr, int lane, int width) {
    int pos = lane * width;
    const uint8_t* p = hdr + (pos >> 3);
    unsigned v = (unsigned)p[0] | ((unsigned)p[1] << 8);
    if (width > 8) v |= (unsigned)p[2] << 16;   // 12/16-bit words may straddle three bytes
    return (v >> (pos & 7)) & ((1u << width) - 1u);
}

// Same, but never reads past hdr[nbytes-1].
__device__ __forceinline__ unsigned load_lane_field_safe(const uint8_t* hdr, int nbytes, int lane, int width) {
    int pos = lane * width;
    int b = pos >> 3;
    unsigned v = 0;
#pragma unroll
    for (int i = 0; i < 3; i++)
        if (b + i < nbytes) v |= (unsigned)hdr[b + i] << (8 * i);
    return (v >> (pos & 7)) & ((1u << width) - 1u);
}

// Warp-cooperative store of the lanes' words (width bits each) as a packed bit string of
// 4*width bytes starting at hdr (any alignment, byte stores).
// Must be called by all 32 lanes (the shuffles are warp-wide).
__device__ __forceinline__ void store_lane_fields(uint8_t* hdr, int lane, int width, unsigned word) {
    const int nbytes = 4 * width;   // 32 lanes * width bits
#pragma unroll
    for (int k = 0; k < 2; k++) {   // width <= 16 -> at most 64 bytes -> two bytes per lane
        int b = lane + 32 * k;
        // byte b covers bits [8b, 8b+8); lane words first..last overlap it (at most 3)
        int first = (8 * b) / width;
        int last = (8 * b + 7) / width;
        unsigned val = 0;
#pragma unroll
        for (int j = 0; j < 3; j++) {
            int l = first + j;
            unsigned wl = __shfl_sync(0xffffffffu, word, l & 31);
            int shift = l * width - 8 * b;
            unsigned piece = shift >= 0 ? (wl << shift) : (wl >> (-shift));
            if (l <= last && l < 32) val |= piece;
        }
        if (b < nbytes) hdr[b] = (uint8_t)(val & 0xFFu);
    }
}

// Same with the width known at compile time: 8- and 16-bit words are stored directly, 12-bit words
// pair up two lanes per three bytes (one shuffle); other widths take the generic routine.
// hdr must be 2-byte aligned.  Must be called by all 32 lanes.
template <int W>
__device__ __forceinline__ void store_lane_fields_w(uint8_t* hdr, int lane, unsigned word) {
    if (W == 8) {
        hdr[lane] = (uint8_t)word;
    } else if (W == 16) {
        *reinterpret_cast<uint16_t*>(hdr + 2 * lane) = (uint16_t)word;
    } else if (W == 12) {
        const unsigned other = __shfl_xor_sync(0xffffffffu, word, 1);
        uint8_t* p = hdr + 3 * (lane >> 1);
        if (lane & 1) {
            p[2] = (uint8_t)(word >> 4);
        } else {
            p[0] = (uint8_t)word;
            p[1] = (uint8_t)((word >> 8) | ((other & 0xFu) << 4));
        }
    } else {
        store_lane_fields(hdr, lane, W, word);
    }
}

// 64-bit window of a byte string at an even byte offset; p must be 2-byte aligned.
__device__ __forceinline__ uint64_t load_u64_align2(const uint8_t* p) {
    const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
    return (uint64_t)q[0] | ((uint64_t)q[1] << 16) | ((uint64_t)q[2] << 32) | ((uint64_t)q[3] << 48);
}

// Same window from SHARED memory with three aligned 32-bit loads and two funnel shifts.  Reads
// the aligned words that contain [p, p+8) (up to 2 bytes before p and 4 bytes past p+8).
__device__ __forceinline__ void load_u64_smem_align2(const uint8_t* p, unsigned& lo, unsigned& hi) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const unsigned* w = reinterpret_cast<const unsigned*>(a & ~(uintptr_t)3);
    const unsigned sh = (unsigned)(a & 2) * 8;      // 0 or 16
    const unsigned w0 = w[0], w1 = w[1], w2 = w[2];
    lo = __funnelshift_r(w0, w1, sh);
    hi = __funnelshift_r(w1, w2, sh);
}

// ---- shared-memory access by 32-bit shared-window address -----------------------------------
// Hot loops address shared memory with 32-bit offsets and explicit ld.shared / st.shared so that
// no 64-bit generic-pointer arithmetic is generated.  The "memory" clobbers keep the compiler from
// moving them across the warp barriers and cp.async waits that order the data.
__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned lds32(unsigned a) {
    unsigned v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ uint4 lds128(unsigned a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ unsigned lds16(unsigned a) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void sts32(unsigned a, unsigned v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void sts16(unsigned a, unsigned short v) { asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"(v) : "memory"); }
__device__ __forceinline__ void sts128(unsigned a, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// lane word of `width` bits (<= 16) at bit lane*width of a header that starts at shared address
// hdr (any alignment): two aligned 32-bit loads and a funnel shift.  May read up to 7 bytes past
// the header.
__device__ __forceinline__ unsigned lds_lane_field(unsigned hdr, int lane, int width) {
    if (width == 16) return lds16(hdr + 2 * lane);     // headers start at even addresses: one aligned load
    const unsigned bit = hdr * 8u + (unsigned)(lane * width);
    const unsigned wa = (bit >> 5) << 2;
    return __funnelshift_r(lds32(wa), lds32(wa + 4), bit & 31u) & ((1u << width) - 1u);
}

// 64-bit window at shared address a (2-byte aligned): three aligned 32-bit loads, two funnel
// shifts.  Reads up to 2 bytes before a and 4 bytes past a+8.
__device__ __forceinline__ void lds_u64_align2(unsigned a, unsigned& lo, unsigned& hi) {
    const unsigned wa = a & ~3u, sh = (a & 2u) * 8u;
    const unsigned w0 = lds32(wa), w1 = lds32(wa + 4), w2 = lds32(wa + 8);
    lo = __funnelshift_r(w0, w1, sh);
    hi = __funnelshift_r(w1, w2, sh);
}

}  // namespace pkv
