// Device helpers shared by the bit-pack kernels (pack.cu, fused_encode.cu).
#pragma once
#include "common.cuh"

namespace pkv {

constexpr int kWarpsPerCta = 4;

// ---- per-pack helpers --------------------------------------------------------------------

// bytewise bit_length of four packed bytes, summed
__device__ __forceinline__ unsigned sum_bitlen4(unsigned d) {
    return bit_length_u32(d & 0xFFu) + bit_length_u32((d >> 8) & 0xFFu) + bit_length_u32((d >> 16) & 0xFFu) +
           bit_length_u32(d >> 24);
}

__device__ __forceinline__ void store_pack_smem(uint8_t* dst, uint64_t w, int len) {
    // dst is 2-byte aligned; the pack takes 2*len bytes = len u16 words
    uint16_t* q = reinterpret_cast<uint16_t*>(dst);
#pragma unroll
    for (int i = 0; i < 4; i++)
        if (i < len) q[i] = (uint16_t)(w >> (16 * i));
}

// Copies `size` bytes from shared `src` to global `dst`; both have the same address modulo
// 16 and are 2-byte aligned.  Warp-cooperative.
__device__ __forceinline__ void warp_copy_out(uint8_t* dst, const uint8_t* src, int size, int lane) {
    int head = (16 - (int)(reinterpret_cast<uintptr_t>(dst) & 15)) & 15;
    if (head > size) head = size;
    for (int i = 2 * lane; i < head; i += 64)
        *reinterpret_cast<uint16_t*>(dst + i) = *reinterpret_cast<const uint16_t*>(src + i);
    int body = (size - head) & ~15;
    for (int i = 16 * lane; i < body; i += 16 * 32)
        *reinterpret_cast<uint4*>(dst + head + i) = *reinterpret_cast<const uint4*>(src + head + i);
    for (int i = head + body + 2 * lane; i < size; i += 64)
        *reinterpret_cast<uint16_t*>(dst + i) = *reinterpret_cast<const uint16_t*>(src + i);
}

}  // namespace pkv
