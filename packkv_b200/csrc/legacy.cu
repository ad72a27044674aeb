// The reference's four stand-alone GPU entry points, kept for callers of the old two-step API
// (evaluation/evaluation.py:398-715): products of q or w with the PACKED codes, and the
// zero-point / scale epilogues.  The fused decode kernel supersedes them on the hot path; these
// are simple warp-per-block kernels that accumulate in fp32 and are deterministic.
//   kq_mat_vec_mul  packkv_cuda_ext/src/kernels.cu:426-630
//   wv_mat_vec_mul  packkv_cuda_ext/src/kernels.cu:632-859
//   fused_kq        packkv_cuda_ext/src/fused_kernels.cu:13-185
//   fused_wv        packkv_cuda_ext/src/fused_kernels.cu:187-370
#include <cooperative_groups.h>

#include "common.cuh"
#include "launch.h"

namespace cg = cooperative_groups;

namespace pkv {

template <typename T> struct LT;
template <> struct LT<__half> {
    static __device__ __forceinline__ float ld(const __half* p) { return __half2float(*p); }
    static __device__ __forceinline__ __half cvt(float x) { return __float2half_rn(x); }
};
template <> struct LT<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ __nv_bfloat16 cvt(float x) { return __float2bfloat16_rn(x); }
};

// copies a block into shared memory keeping the 16-byte phase; returns the mirror of src
__device__ __forceinline__ const uint8_t* stage_block(uint8_t* sbuf, const uint8_t* src, int size, int lane,
                                                      const uint8_t* lo, const uint8_t* hi) {
    const int phase = (int)(reinterpret_cast<uintptr_t>(src) & 15);
    const uint8_t* a = src - phase;
    const int total = (phase + size + 15) & ~15;
    for (int i = 16 * lane; i < total; i += 512) {
        const uint8_t* p = a + i;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (p >= lo && p + 16 <= hi) v = *reinterpret_cast<const uint4*>(p);
        else {
            unsigned q[4] = {0, 0, 0, 0};
            for (int b = 0; b < 16; b++)
                if (p + b >= lo && p + b < hi) q[b >> 2] |= (unsigned)p[b] << (8 * (b & 3));
            v = make_uint4(q[0], q[1], q[2], q[3]);
        }
        *reinterpret_cast<uint4*>(sbuf + i) = v;
    }
    return sbuf + phase;
}

// t[h, n] = sum_d q[h, d] * code[n, h*128 + d]; q arrives in the reference's lane-permuted order:
// first 64 entries = (q[4l], q[4l+1]) for l = 0..31, last 64 = (q[4l+2], q[4l+3]).
template <typename T>
__global__ void __launch_bounds__(128) kq_kernel(LegacyArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    const int64_t blk_id = (int64_t)blockIdx.x * 4 + wic;
    const int nhid = a.hidden / 128, nctx = a.ctx_len / a.cb;
    if (blk_id >= (int64_t)nctx * nhid) return;
    const int cbi = (int)(blk_id / nhid), hbi = (int)(blk_id % nhid);
    const int rounds = a.cb / 16, lb = len_field_bits(a.bits);
    const int bound = 2 * rounds + rounds * (16 * a.bits + 16 * lb + 256 * a.bits);
    const int slot = (bound + 48 + 15) & ~15;
    const unsigned off = a.info[2 * blk_id], size = a.info[2 * blk_id + 1];
    if ((int64_t)off + size > a.stream_bytes || (int)size > bound || size < 4) {
        if (lane == 0) atomicOr(a.flags, kFlagBadStream);
        return;
    }
    const uint8_t* blk = stage_block(smem + wic * slot, a.stream + off, (int)size, lane, a.stream, a.stream + a.stream_bytes);
    __syncwarp();
    const T* q = reinterpret_cast<const T*>(a.vec) + hbi * 128;
    const float q0 = LT<T>::ld(q + 2 * lane), q1 = LT<T>::ld(q + 2 * lane + 1), q2 = LT<T>::ld(q + 64 + 2 * lane), q3 = LT<T>::ld(q + 64 + 2 * lane + 1);
    T* out = reinterpret_cast<T*>(a.out) + (int64_t)hbi * a.ctx_len + (int64_t)cbi * a.cb;
    int pos = 2 * rounds;
    for (int r = 0; r < rounds; r++) {
        const uint8_t* hdr = blk + pos;
        const unsigned minword = load_lane_field(hdr, lane, 4 * a.bits);
        const unsigned lenword = load_lane_field(hdr + 16 * a.bits, lane, 4 * lb);
        unsigned lens4 = 0;
        int len[4];
        for (int j = 0; j < 4; j++) { len[j] = min((int)((lenword >> (j * lb)) & ((1u << lb) - 1u)), 4); lens4 |= (unsigned)len[j] << (8 * j); }
        const unsigned inc = warp_inclusive_sum(lens4);
        const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
        const unsigned exc = inc - lens4;
        const uint8_t* packs = hdr + 16 * a.bits + 16 * lb;
        unsigned before = 0;
        uint64_t w[4];
        unsigned mn[4];
        for (int j = 0; j < 4; j++) {
            w[j] = load_u64_align2(packs + 2 * (before + ((exc >> (8 * j)) & 0xFFu)));
            before += (tot >> (8 * j)) & 0xFFu;
            mn[j] = (minword >> (j * a.bits)) & ((1u << a.bits) - 1u);
        }
        const float qs[4] = {q0, q1, q2, q3};
        float mine = 0.f;   // lane t (< 16) keeps the score of token t
        for (int t = 0; t < 16; t++) {
            float d = 0.f;
            for (int j = 0; j < 4; j++) {
                const unsigned c = ((unsigned)(w[j] >> (len[j] * (15 - t))) & ((1u << len[j]) - 1u)) + mn[j];
                d += qs[j] * (float)c;
            }
            for (int s = 16; s > 0; s >>= 1) d += __shfl_xor_sync(0xffffffffu, d, s);
            if (lane == t) mine = d;
        }
        if (lane < 16) out[r * 16 + lane] = LT<T>::cvt(mine);
        pos += 16 * a.bits + 16 * lb + 2 * (int)before;
    }
}

// out[hb*64 + c] += sum_n w[h, n] * code[n, hb*64 + c], h = hb*64/128.  One cluster of kWvSlices CTAs per
// 64-channel block column: the CTAs' 8 warps each stride over the token blocks; warps, then CTAs (through
// distributed shared memory, on the cluster's first CTA) are summed in a fixed order.
constexpr int kWvSlices = 8;
template <typename T>
__global__ void __launch_bounds__(256) wv_kernel(LegacyArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ float part[8][64];
    __shared__ float csum[64];
    cg::cluster_group cluster = cg::this_cluster();
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    const int hbi = blockIdx.x / kWvSlices, slice = (int)cluster.block_rank();
    const int nhid = a.hidden / 64, nctx = a.ctx_len / a.cb;
    const VGeom g(a.cb, a.bits);
    const int lb = len_field_bits(a.bits);
    const int bound = g.head_bytes + g.nseg * (g.min_bytes + g.len_bytes + 32 * g.ppt * 2 * a.bits);
    const int slot = (bound + 48 + 15) & ~15;
    const T* wrow = reinterpret_cast<const T*>(a.vec) + (int64_t)(hbi * 64 / 128) * a.ctx_len;
    float acc0 = 0.f, acc1 = 0.f;   // channels lane and 32 + lane
    for (int cbi = slice * 8 + wic; cbi < nctx; cbi += 8 * kWvSlices) {
        const int64_t blk_id = (int64_t)cbi * nhid + hbi;
        const unsigned off = a.info[2 * blk_id], size = a.info[2 * blk_id + 1];
        if ((int64_t)off + size > a.stream_bytes || (int)size > bound || size < 4) {
            if (lane == 0) atomicOr(a.flags, kFlagBadStream);
            continue;
        }
        __syncwarp();
        const uint8_t* blk = stage_block(smem + wic * slot, a.stream + off, (int)size, lane, a.stream, a.stream + a.stream_bytes);
        __syncwarp();
        int pos = g.head_bytes;
        for (int w = 0; w < 2; w++)
            for (int r = 0; r < g.rpw; r++) {
                const uint8_t* hdr = blk + pos;
                const unsigned minword = load_lane_field(hdr, lane, g.ppt * a.bits);
                const unsigned lenword = load_lane_field(hdr + g.min_bytes, lane, g.ppt * lb);
                unsigned lens4 = 0;
                int len[4];
                for (int q = 0; q < 4; q++) { len[q] = q < g.ppt ? min((int)((lenword >> (q * lb)) & ((1u << lb) - 1u)), 4) : 0; lens4 |= (unsigned)len[q] << (8 * q); }
                const unsigned inc = warp_inclusive_sum(lens4);
                const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
                const unsigned exc = inc - lens4;
                const uint8_t* packs = hdr + g.min_bytes + g.len_bytes;
                unsigned before = 0;
                float s = 0.f;
                for (int q = 0; q < g.ppt; q++) {
                    const uint64_t wd = load_u64_align2(packs + 2 * (before + ((exc >> (8 * q)) & 0xFFu)));
                    before += (tot >> (8 * q)) & 0xFFu;
                    const unsigned mn = (minword >> (q * a.bits)) & ((1u << a.bits) - 1u);
                    const T* wt = wrow + (int64_t)cbi * a.cb + (r * g.ppt + q) * 16;
                    for (int t = 0; t < 16; t++) {
                        const unsigned c = ((unsigned)(wd >> (len[q] * (15 - t))) & ((1u << len[q]) - 1u)) + mn;
                        s += LT<T>::ld(wt + t) * (float)c;
                    }
                }
                if (w == 0) acc0 += s; else acc1 += s;
                pos += g.min_bytes + g.len_bytes + 2 * (int)before;
            }
    }
    part[wic][lane] = acc0;
    part[wic][32 + lane] = acc1;
    __syncthreads();
    if (threadIdx.x < 64) {
        float s = 0.f;
        for (int w = 0; w < 8; w++) s += part[w][threadIdx.x];
        csum[threadIdx.x] = s;
    }
    cluster.sync();
    if (slice == 0 && threadIdx.x < 64) {
        float s = 0.f;
        for (int r = 0; r < kWvSlices; r++) s += cluster.map_shared_rank(csum, r)[threadIdx.x];
        reinterpret_cast<float*>(a.out)[hbi * 64 + threadIdx.x] += s;
    }
    cluster.sync();   // the other CTAs' sums stay alive until the first one has read them
}

// our_kq[m, n] = (sum_d q[m, d] * zero[n] + t[m, n]) * scale[n]
template <typename T>
__global__ void __launch_bounds__(256) fused_kq_kernel(T* out, const T* q, const T* zero, const T* scale, const T* t, int M, int N, int K) {
    __shared__ float red[8];
    const int m = blockIdx.x;
    float s = 0.f;
    for (int d = threadIdx.x; d < K; d += 256) s += LT<T>::ld(q + (int64_t)m * K + d);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    float qs = 0.f;
    for (int w = 0; w < 8; w++) qs += red[w];
    for (int n = threadIdx.x; n < N; n += 256) {
        const float u = qs * LT<T>::ld(zero + n) + LT<T>::ld(t + (int64_t)m * N + n);
        out[(int64_t)m * N + n] = LT<T>::cvt(u * LT<T>::ld(scale + n));
    }
}

// our_wv[m, d] = sum_n w[m, n] * zero[n] * scale[n] + term1[m, d]
template <typename T>
__global__ void __launch_bounds__(256) fused_wv_kernel(T* out, const T* w, const T* zero, const T* scale, const T* term1, int M, int N, int D) {
    __shared__ float red[8];
    const int m = blockIdx.x;
    float s = 0.f;
    for (int n = threadIdx.x; n < N; n += 256) s += LT<T>::ld(w + (int64_t)m * N + n) * LT<T>::ld(zero + n) * LT<T>::ld(scale + n);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    float ws = 0.f;
    for (int i = 0; i < 8; i++) ws += red[i];
    for (int d = threadIdx.x; d < D; d += 256) out[(int64_t)m * D + d] = LT<T>::cvt(ws + LT<T>::ld(term1 + (int64_t)m * D + d));
}

int launch_legacy_matvec(bool is_k, const LegacyArgs& a, cudaStream_t st) {
    if (a.bits < 2 || a.bits > 4) return kUnsupported;
    if (is_k ? (a.hb != 128 || (a.cb != 32 && a.cb != 64 && a.cb != 128)) : (a.hb != 64 || (a.cb != 32 && a.cb != 64 && a.cb != 128))) return kUnsupported;
    if (a.ctx_len <= 0 || a.hidden <= 0 || a.ctx_len % a.cb || a.hidden % 128) return kBadArgument;
    if (!a.stream || !a.info || !a.vec || !a.out || !a.flags) return kBadArgument;
    if (reinterpret_cast<uintptr_t>(a.stream) & 15) return kBadArgument;
    if (is_k) {
        const int rounds = a.cb / 16, lb = len_field_bits(a.bits);
        const int slot = (2 * rounds + rounds * (16 * a.bits + 16 * lb + 256 * a.bits) + 48 + 15) & ~15;
        const int64_t nblk = (int64_t)(a.ctx_len / a.cb) * (a.hidden / 128);
        if (a.is_bf16) kq_kernel<__nv_bfloat16><<<(unsigned)((nblk + 3) / 4), 128, 4 * slot, st>>>(a);
        else kq_kernel<__half><<<(unsigned)((nblk + 3) / 4), 128, 4 * slot, st>>>(a);
    } else {
        const VGeom g(a.cb, a.bits);
        const int slot = (g.head_bytes + g.nseg * (g.min_bytes + g.len_bytes + 32 * g.ppt * 2 * a.bits) + 48 + 15) & ~15;
        const int smem = 8 * slot;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(a.hidden / 64) * kWvSlices, 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = kWvSlices; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = a.is_bf16 ? cudaLaunchKernelEx(&cfg, wv_kernel<__nv_bfloat16>, a) : cudaLaunchKernelEx(&cfg, wv_kernel<__half>, a);
        if (e != cudaSuccess) { cudaGetLastError(); return kCudaError; }
    }
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

int launch_fused_epilogue(bool is_kq, void* out, const void* a, const void* zero, const void* scale, const void* t,
                          int M, int N, int K, int is_bf16, cudaStream_t st) {
    if (M <= 0 || N <= 0 || K <= 0 || !out || !a || !zero || !scale || !t) return kBadArgument;
    if (is_bf16) {
        using T = __nv_bfloat16;
        if (is_kq) fused_kq_kernel<T><<<M, 256, 0, st>>>((T*)out, (const T*)a, (const T*)zero, (const T*)scale, (const T*)t, M, N, K);
        else fused_wv_kernel<T><<<M, 256, 0, st>>>((T*)out, (const T*)a, (const T*)zero, (const T*)scale, (const T*)t, M, N, K);
    } else {
        using T = __half;
        if (is_kq) fused_kq_kernel<T><<<M, 256, 0, st>>>((T*)out, (const T*)a, (const T*)zero, (const T*)scale, (const T*)t, M, N, K);
        else fused_wv_kernel<T><<<M, 256, 0, st>>>((T*)out, (const T*)a, (const T*)zero, (const T*)scale, (const T*)t, M, N, K);
    }
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

}  // namespace pkv
