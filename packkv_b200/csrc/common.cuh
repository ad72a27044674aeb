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
        unsigned n = __shfl_up_sync(0xffffffffu, v, d);
        if ((int)lane_id() >= d) v += n;
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

// 64-bit window of a byte string at an even byte offset; p must be 2-byte aligned.
__device__ __forceinline__ uint64_t load_u64_align2(const uint8_t* p) {
    const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
    return (uint64_t)q[0] | ((uint64_t)q[1] << 16) | ((uint64_t)q[2] << 32) | ((uint64_t)q[3] << 48);
}

}  // namespace pkv
