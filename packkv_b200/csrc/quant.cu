// Block quantiser: fp16/bf16 K or V -> uint8 codes + scale + zero-point, bit-identical to the
// reference's PyTorch arithmetic (utils/compute.py:84-112), which rounds to the tensor dtype
// after every op:
//     scale = (max - min) * rel
//     zero  = round(min / scale);  code = round(x / scale) - zero            (default)
//     zero  = min;                 code = round((x - min) / scale)           (high-precision zero)
// Each op below is done in fp32 (exactly what PyTorch's half/bfloat16 kernels do) and rounded
// back with round-to-nearest-even; round() is round-half-to-even.
//
// Modes (reduction set of one scale/zero pair, reference QUANT_DIM, utils/compute.py:405-410):
//   channel: one (sequence, kv head, token block, channel)        -> params (B, H, n_blocks, 128)
//   token  : one (sequence, token) across all heads and channels  -> params (B, n_tokens)
//   vector : one (sequence, kv head, token) across its channels    -> params (B, H, n_tokens)
//   block  : one (sequence, token block) across heads and channels -> params (B, n_blocks)
// Channel and token are the modes of the reference's two quantisation methods and the only ones the
// encoder's single pass and the attention kernel take; vector and block exist in the reference's enum and
// are served by this quantiser, pkv_dequantize and the codec entry points on the code matrix.
// Codes are written as the codec's input matrix: (B, S, H*128) uint8, row = token.
#include "common.cuh"
#include "launch.h"
#include "quant_dev.cuh"

namespace pkv {

// grid (n_blocks, H, B), 128 threads: thread = channel
template <typename T, bool HP>
__global__ void __launch_bounds__(128) quant_channel_kernel(QuantArgs q) {
    const int nb = blockIdx.x, h = blockIdx.y, b = blockIdx.z, d = threadIdx.x;
    const T* x = reinterpret_cast<const T*>(q.x) + (int64_t)b * q.stride_b + (int64_t)h * q.stride_h + (int64_t)nb * q.block * q.stride_s + d;
    float lo = INFINITY, hi = -INFINITY;
    for (int t = 0; t < q.block; t++) {
        const float v = QT<T>::ld(x + (int64_t)t * q.stride_s);
        lo = fminf(lo, v); hi = fmaxf(hi, v);
    }
    const Quantiser<T, HP> qz(lo, hi, q.rel);
    const float limit = q.bits > 0 ? (float)(1 << q.bits) : 256.f;
    bool bad = false;
    uint8_t* out = q.codes + (int64_t)b * q.codes_seq_stride + (int64_t)nb * q.block * (q.heads * 128) + h * 128 + d;
    for (int t = 0; t < q.block; t++) {
        const float v = QT<T>::ld(x + (int64_t)t * q.stride_s);
        out[(int64_t)t * (q.heads * 128)] = (uint8_t)code_byte(qz.code(v), limit, bad);
    }
    const int64_t pi = (((int64_t)b * q.heads + h) * q.param_blocks + q.first_block + nb) * 128 + d;
    reinterpret_cast<T*>(q.scale)[pi] = QT<T>::cvt(qz.scale);
    reinterpret_cast<T*>(q.zero)[pi] = QT<T>::cvt(qz.zero);
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(q.flags, kFlagCodeRange);
}

// one warp per (sequence, token); lane owns 4 channels of every head
template <typename T, bool HP>
__global__ void __launch_bounds__(128) quant_token_kernel(QuantArgs q) {
    const int lane = lane_id();
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= (int64_t)q.batch * q.tokens) return;
    const int b = (int)(row / q.tokens), t = (int)(row % q.tokens);
    const T* x = reinterpret_cast<const T*>(q.x) + (int64_t)b * q.stride_b + (int64_t)t * q.stride_s + 4 * lane;
    float lo = INFINITY, hi = -INFINITY;
    for (int h = 0; h < q.heads; h++) {
        const uint2 raw = *reinterpret_cast<const uint2*>(x + (int64_t)h * q.stride_h);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; j++) { const float v = QT<T>::ld(e + j); lo = fminf(lo, v); hi = fmaxf(hi, v); }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, s));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, s));
    }
    const Quantiser<T, HP> qz(lo, hi, q.rel);
    const float limit = q.bits > 0 ? (float)(1 << q.bits) : 256.f;
    bool bad = false;
    uint8_t* out = q.codes + (int64_t)b * q.codes_seq_stride + (int64_t)t * (q.heads * 128) + 4 * lane;
    for (int h = 0; h < q.heads; h++) {
        const uint2 raw = *reinterpret_cast<const uint2*>(x + (int64_t)h * q.stride_h);
        const T* e = reinterpret_cast<const T*>(&raw);
        unsigned u = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) u |= code_byte(qz.code(QT<T>::ld(e + j)), limit, bad) << (8 * j);
        *reinterpret_cast<unsigned*>(out + h * 128) = u;
    }
    if (lane == 0) {
        const int64_t pi = (int64_t)b * q.param_tokens + q.first_token + t;
        reinterpret_cast<T*>(q.scale)[pi] = QT<T>::cvt(qz.scale);
        reinterpret_cast<T*>(q.zero)[pi] = QT<T>::cvt(qz.zero);
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(q.flags, kFlagCodeRange);
}

// one warp per (sequence, head, token); lane owns 4 channels
template <typename T, bool HP>
__global__ void __launch_bounds__(128) quant_vector_kernel(QuantArgs q) {
    const int lane = lane_id();
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= (int64_t)q.batch * q.heads * q.tokens) return;
    const int t = (int)(row % q.tokens), h = (int)((row / q.tokens) % q.heads), b = (int)(row / ((int64_t)q.tokens * q.heads));
    const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const T*>(q.x) + (int64_t)b * q.stride_b + (int64_t)h * q.stride_h +
                                                      (int64_t)t * q.stride_s + 4 * lane);
    const T* e = reinterpret_cast<const T*>(&raw);
    float lo = INFINITY, hi = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; j++) { const float v = QT<T>::ld(e + j); lo = fminf(lo, v); hi = fmaxf(hi, v); }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, s));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, s));
    }
    const Quantiser<T, HP> qz(lo, hi, q.rel);
    const float limit = q.bits > 0 ? (float)(1 << q.bits) : 256.f;
    bool bad = false;
    unsigned u = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) u |= code_byte(qz.code(QT<T>::ld(e + j)), limit, bad) << (8 * j);
    *reinterpret_cast<unsigned*>(q.codes + (int64_t)b * q.codes_seq_stride + (int64_t)t * (q.heads * 128) + h * 128 + 4 * lane) = u;
    if (lane == 0) {
        const int64_t pi = ((int64_t)b * q.heads + h) * q.param_tokens + q.first_token + t;
        reinterpret_cast<T*>(q.scale)[pi] = QT<T>::cvt(qz.scale);
        reinterpret_cast<T*>(q.zero)[pi] = QT<T>::cvt(qz.zero);
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(q.flags, kFlagCodeRange);
}

// grid (n_blocks, B), 256 threads: one pair of parameters for block tokens x all heads x 128 channels
template <typename T, bool HP>
__global__ void __launch_bounds__(256) quant_block_kernel(QuantArgs q) {
    __shared__ float red[2][8];
    const int nb = blockIdx.x, b = blockIdx.y, lane = lane_id(), wic = threadIdx.x >> 5;
    const T* xb = reinterpret_cast<const T*>(q.x) + (int64_t)b * q.stride_b + (int64_t)nb * q.block * q.stride_s;
    const int units = q.block * q.heads * 32;                    // 4 channels each
    float lo = INFINITY, hi = -INFINITY;
    for (int u = threadIdx.x; u < units; u += 256) {
        const int c4 = u & 31, h = (u >> 5) % q.heads, t = (u >> 5) / q.heads;
        const uint2 raw = *reinterpret_cast<const uint2*>(xb + (int64_t)h * q.stride_h + (int64_t)t * q.stride_s + 4 * c4);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; j++) { const float v = QT<T>::ld(e + j); lo = fminf(lo, v); hi = fmaxf(hi, v); }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, s));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, s));
    }
    if (lane == 0) { red[0][wic] = lo; red[1][wic] = hi; }
    __syncthreads();
#pragma unroll
    for (int w = 0; w < 8; w++) { lo = fminf(lo, red[0][w]); hi = fmaxf(hi, red[1][w]); }
    const Quantiser<T, HP> qz(lo, hi, q.rel);
    const float limit = q.bits > 0 ? (float)(1 << q.bits) : 256.f;
    bool bad = false;
    uint8_t* ob = q.codes + (int64_t)b * q.codes_seq_stride + (int64_t)nb * q.block * (q.heads * 128);
    for (int u = threadIdx.x; u < units; u += 256) {
        const int c4 = u & 31, h = (u >> 5) % q.heads, t = (u >> 5) / q.heads;
        const uint2 raw = *reinterpret_cast<const uint2*>(xb + (int64_t)h * q.stride_h + (int64_t)t * q.stride_s + 4 * c4);
        const T* e = reinterpret_cast<const T*>(&raw);
        unsigned w4 = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) w4 |= code_byte(qz.code(QT<T>::ld(e + j)), limit, bad) << (8 * j);
        *reinterpret_cast<unsigned*>(ob + (int64_t)t * (q.heads * 128) + h * 128 + 4 * c4) = w4;
    }
    if (threadIdx.x == 0) {
        const int64_t pi = (int64_t)b * q.param_blocks + q.first_block + nb;
        reinterpret_cast<T*>(q.scale)[pi] = QT<T>::cvt(qz.scale);
        reinterpret_cast<T*>(q.zero)[pi] = QT<T>::cvt(qz.zero);
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(q.flags, kFlagCodeRange);
}

template <typename T, bool HP>
static void launch_q(const QuantArgs& q, cudaStream_t st) {
    if (q.mode == 2) {
        const int64_t rows = (int64_t)q.batch * q.heads * q.tokens;
        quant_vector_kernel<T, HP><<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(q);
    } else if (q.mode == 3) {
        quant_block_kernel<T, HP><<<dim3(q.tokens / q.block, q.batch), 256, 0, st>>>(q);
    } else if (q.mode == 0) {
        dim3 grid(q.tokens / q.block, q.heads, q.batch);
        quant_channel_kernel<T, HP><<<grid, 128, 0, st>>>(q);
    } else {
        const int64_t rows = (int64_t)q.batch * q.tokens;
        quant_token_kernel<T, HP><<<(unsigned)((rows + 3) / 4), 128, 0, st>>>(q);
    }
}

int launch_quantize(const QuantArgs& q, cudaStream_t st) {
    if (q.batch < 0 || q.heads <= 0 || q.tokens < 0 || q.block <= 0 || q.tokens % q.block) return kBadArgument;
    if (q.mode < 0 || q.mode > 3) return kUnsupported;
    if (q.bits < 0 || q.bits > 8) return kBadArgument;
    if ((int64_t)q.batch * q.tokens == 0) return kOk;
    if (!q.x || !q.codes || !q.scale || !q.zero || !q.flags) return kBadArgument;
    if ((reinterpret_cast<uintptr_t>(q.x) & 7) || (q.stride_b & 3) || (q.stride_h & 3) || (q.stride_s & 3)) return kBadArgument;
    if ((reinterpret_cast<uintptr_t>(q.codes) & 3) || (q.codes_seq_stride & 3)) return kBadArgument;
    if (q.is_bf16) { if (q.high_precision_zero) launch_q<__nv_bfloat16, true>(q, st); else launch_q<__nv_bfloat16, false>(q, st); }
    else           { if (q.high_precision_zero) launch_q<__half, true>(q, st); else launch_q<__half, false>(q, st); }
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

}  // namespace pkv
