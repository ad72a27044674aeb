// In-block token reordering (the reference's median_repacking, utils/compute.py:262-270).
//   key[token]  = lower median of the token's V codes over all heads and channels
//   order       = tokens of a block sorted by key, descending
// The reference sorts with torch.sort(descending=True), which leaves the order of equal keys
// unspecified; here ties keep their original order (stable), so the result is deterministic.
// Attention does not depend on the order of tokens inside a block, so K and V rows and the
// per-token parameters are simply gathered by `order` before packing.
#include "common.cuh"
#include "launch.h"

namespace pkv {

// grid (n_blocks, batch); one warp per token, CTA of `block` tokens handled by 8 warps in turns
__global__ void __launch_bounds__(256) median_order_kernel(ReorderArgs a) {
    __shared__ unsigned char key[128];
    const int blk = blockIdx.x, b = blockIdx.y;
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    const int row_bytes = a.heads * 128;
    const int need = (row_bytes + 1) / 2;            // lower median: smallest m with count(<= m) >= ceil(n/2)
    for (int t = wic; t < a.block; t += 8) {
        const uint8_t* row = a.v_codes + (int64_t)b * a.codes_seq_stride + (int64_t)(blk * a.block + t) * row_bytes;
        unsigned cnt[8];                              // two 16-bit counters per word: thresholds 2i and 2i+1
#pragma unroll
        for (int i = 0; i < 8; i++) cnt[i] = 0;
        for (int off = lane * 16; off < row_bytes; off += 512) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + off));
            const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 8; i++) {
                unsigned c0 = 0, c1 = 0;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    c0 += __popc(__vcmpleu4(w[k], 0x01010101u * (2 * i))) >> 3;
                    c1 += __popc(__vcmpleu4(w[k], 0x01010101u * (2 * i + 1))) >> 3;
                }
                cnt[i] += c0 | (c1 << 16);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) cnt[i] += __shfl_xor_sync(0xffffffffu, cnt[i], s);
        int med = 16;                                  // codes above 15 are not expected (bits <= 4)
#pragma unroll
        for (int i = 7; i >= 0; i--) {
            if ((int)(cnt[i] >> 16) >= need) med = 2 * i + 1;
            if ((int)(cnt[i] & 0xFFFFu) >= need) med = 2 * i;
        }
        if (lane == 0) {
            key[t] = (unsigned char)med;
            if (a.keys) a.keys[(int64_t)b * a.tokens + blk * a.block + t] = (uint8_t)med;
        }
    }
    __syncthreads();
    const int i = threadIdx.x;
    if (i < a.block) {
        const int ki = key[i];
        int rank = 0;
        for (int j = 0; j < a.block; j++) {
            const int kj = key[j];
            rank += (kj > ki) || (kj == ki && j < i);
        }
        a.order[((int64_t)b * (a.tokens / a.block) + blk) * a.block + rank] = (uint8_t)i;
    }
}

// dst row r of a block <- src row order[r]; rows of `row_bytes` bytes (multiple of 16). grid (tokens, batch)
__global__ void __launch_bounds__(64) gather_rows_kernel(const uint8_t* src, uint8_t* dst, int64_t seq_stride, const uint8_t* order,
                                                         int tokens, int block, int row_bytes) {
    const int t = blockIdx.x, b = blockIdx.y;
    const int blk = t / block, r = t - blk * block;
    const int from = blk * block + order[((int64_t)b * (tokens / block) + blk) * block + r];
    const uint4* s = reinterpret_cast<const uint4*>(src + (int64_t)b * seq_stride + (int64_t)from * row_bytes);
    uint4* d = reinterpret_cast<uint4*>(dst + (int64_t)b * seq_stride + (int64_t)t * row_bytes);
    for (int i = threadIdx.x; i < row_bytes / 16; i += 64) d[i] = __ldg(s + i);
}

// per-token 16-bit parameters (scale / zero): dst[b][first + t] <- src[b][first + blockstart + order]
__global__ void __launch_bounds__(128) gather_params_kernel(const uint16_t* src, uint16_t* dst, int64_t row_len, int first,
                                                            const uint8_t* order, int tokens, int block) {
    const int blk = blockIdx.x, b = blockIdx.y, r = threadIdx.x;
    if (r >= block) return;
    const int from = blk * block + order[((int64_t)b * (tokens / block) + blk) * block + r];
    dst[(int64_t)b * row_len + first + blk * block + r] = src[(int64_t)b * row_len + first + from];
}

int launch_median_order(const ReorderArgs& a, cudaStream_t st) {
    if (a.batch < 0 || a.heads <= 0 || a.tokens < 0 || a.block <= 0 || a.block > 128 || a.tokens % a.block) return kBadArgument;
    if ((int64_t)a.batch * a.tokens == 0) return kOk;
    if (!a.v_codes || !a.order || (reinterpret_cast<uintptr_t>(a.v_codes) & 15) || (a.codes_seq_stride & 15)) return kBadArgument;
    median_order_kernel<<<dim3(a.tokens / a.block, a.batch), 256, 0, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

int launch_gather_rows(const uint8_t* src, uint8_t* dst, int64_t seq_stride, const uint8_t* order, int batch, int tokens,
                       int block, int row_bytes, cudaStream_t st) {
    if (batch < 0 || tokens < 0 || block <= 0 || tokens % block || row_bytes <= 0 || row_bytes % 16) return kBadArgument;
    if ((int64_t)batch * tokens == 0) return kOk;
    if (!src || !dst || !order || src == dst) return kBadArgument;
    gather_rows_kernel<<<dim3(tokens, batch), 64, 0, st>>>(src, dst, seq_stride, order, tokens, block, row_bytes);
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

int launch_gather_params(const void* src, void* dst, int64_t row_len, int first, const uint8_t* order, int batch, int tokens,
                         int block, cudaStream_t st) {
    if (batch < 0 || tokens < 0 || block <= 0 || block > 128 || tokens % block) return kBadArgument;
    if ((int64_t)batch * tokens == 0) return kOk;
    if (!src || !dst || !order || src == dst) return kBadArgument;
    gather_params_kernel<<<dim3(tokens / block, batch), 128, 0, st>>>(static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst),
                                                                      row_len, first, order, tokens, block);
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

}  // namespace pkv
