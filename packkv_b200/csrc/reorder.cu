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

// ------------------------------------------------------------------------------------ greedy
// The reference's greedy_repacking (utils/compute.py:210-260) for one block of `block` tokens whose
// feature vector is the token's K codes followed by its V codes (2 * heads * 128 features):
//   for every pack: seed = the remaining token most similar (cosine) to the rounded mean of the
//   remaining tokens, then pack_len-1 times the remaining token that adds the fewest bits,
//   bits = sum over features of bit_length(max - min) of the pack so far; ties take the first
//   remaining token.  The output lists the tokens pack after pack in the order they were picked.
// All comparisons are made in exact integer arithmetic: the cosine argmax compares
// dot_i^2 / |x_i|^2 by cross-multiplication (the mean vector's norm is common to all candidates and
// dots are non-negative), the mean is sum/n rounded half to even.  The reference evaluates the
// same quantities in fp32, so the two agree except where two candidates' cosines differ by less
// than fp32 rounding.
// One CTA (8 warps) per (block, sequence); a warp scores one candidate at a time.
struct GreedyArgs {
    const uint8_t* k_codes;
    const uint8_t* v_codes;
    int64_t seq_stride;     // bytes between sequences in both code matrices
    uint8_t* order;         // (batch, tokens/block, block)
    int tokens, block, pack_len, hidden;
};

__device__ __forceinline__ unsigned bitlen_sum4(unsigned mx, unsigned mn, unsigned x) {
    unsigned s = 0;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const unsigned a = (mx >> (8 * k)) & 0xFFu, b = (mn >> (8 * k)) & 0xFFu, c = (x >> (8 * k)) & 0xFFu;
        s += 32 - __clz(max(a, c) - min(b, c));
    }
    return s;
}

__global__ void __launch_bounds__(256) greedy_order_kernel(GreedyArgs a) {
    extern __shared__ __align__(16) uint8_t gsm[];
    const int blk = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, wic = tid >> 5;
    const int words = a.hidden / 2;                    // 32-bit words per feature vector (K then V)
    const int kwords = a.hidden / 4;
    unsigned* mn = reinterpret_cast<unsigned*>(gsm);   // [words] running min of the pack, 4 features per word
    unsigned* mx = mn + words;                         // [words]
    unsigned* mean = mx + words;                       // [words]
    unsigned short* sum = reinterpret_cast<unsigned short*>(mean + words);   // [4*words] sums over the remaining tokens
    unsigned* score = reinterpret_cast<unsigned*>(sum + 4 * words);           // [128] dot or bit count per candidate
    unsigned* nrm = score + 128;                                              // [128] |x|^2 per token
    __shared__ unsigned char rem[128];
    __shared__ unsigned char out[128];
    __shared__ int pick_s;
    const uint8_t* kb = a.k_codes + (int64_t)b * a.seq_stride + (int64_t)blk * a.block * a.hidden;
    const uint8_t* vb = a.v_codes + (int64_t)b * a.seq_stride + (int64_t)blk * a.block * a.hidden;
    auto word_of = [&](int tok, int w) -> unsigned {
        return w < kwords ? __ldg(reinterpret_cast<const unsigned*>(kb + (int64_t)tok * a.hidden) + w)
                          : __ldg(reinterpret_cast<const unsigned*>(vb + (int64_t)tok * a.hidden) + (w - kwords));
    };
    for (int w = tid; w < words; w += 256) {
        unsigned s0 = 0, s1 = 0, s2 = 0, s3 = 0;
        for (int t = 0; t < a.block; t++) {
            const unsigned x = word_of(t, w);
            s0 += x & 0xFFu; s1 += (x >> 8) & 0xFFu; s2 += (x >> 16) & 0xFFu; s3 += x >> 24;
        }
        sum[4 * w] = (unsigned short)s0; sum[4 * w + 1] = (unsigned short)s1; sum[4 * w + 2] = (unsigned short)s2; sum[4 * w + 3] = (unsigned short)s3;
    }
    for (int t = wic; t < a.block; t += 8) {
        unsigned n = 0;
        for (int w = lane; w < words; w += 32) { const unsigned x = word_of(t, w); n = __dp4a(x, x, n); }
        n = warp_sum(n);
        if (lane == 0) nrm[t] = n;
    }
    if (tid < a.block) rem[tid] = (unsigned char)tid;
    __syncthreads();
    int n_rem = a.block, n_out = 0;
    const int packs = a.block / a.pack_len;
    // removes candidate position s from the list, updates the running sums / pack range
    auto take = [&](int s, bool seed) {
        const int tok = rem[s];
        __syncthreads();
        if (tid == 0) out[n_out] = (unsigned char)tok;
        unsigned char nxt = (tid >= s && tid < n_rem - 1) ? rem[tid + 1] : 0;
        __syncthreads();
        if (tid >= s && tid < n_rem - 1) rem[tid] = nxt;
        for (int w = tid; w < words; w += 256) {
            const unsigned x = word_of(tok, w);
            sum[4 * w] -= x & 0xFFu; sum[4 * w + 1] -= (x >> 8) & 0xFFu; sum[4 * w + 2] -= (x >> 16) & 0xFFu; sum[4 * w + 3] -= x >> 24;
            if (seed) { mn[w] = x; mx[w] = x; }
            else {
                unsigned lo = 0, hi = 0;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const unsigned c = (x >> (8 * k)) & 0xFFu;
                    lo |= min((mn[w] >> (8 * k)) & 0xFFu, c) << (8 * k);
                    hi |= max((mx[w] >> (8 * k)) & 0xFFu, c) << (8 * k);
                }
                mn[w] = lo; mx[w] = hi;
            }
        }
        n_rem--; n_out++;
        __syncthreads();
    };
    for (int p = 0; p < packs; p++) {
        // rounded mean of the remaining tokens
        for (int w = tid; w < words; w += 256) {
            unsigned m = 0;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const unsigned sv = sum[4 * w + k];
                unsigned q = sv / n_rem;
                const unsigned r2 = 2 * (sv - q * n_rem);
                q += (r2 > (unsigned)n_rem) || (r2 == (unsigned)n_rem && (q & 1u));
                m |= q << (8 * k);
            }
            mean[w] = m;
        }
        __syncthreads();
        for (int c = wic; c < n_rem; c += 8) {
            const int tok = rem[c];
            unsigned d = 0;
            for (int w = lane; w < words; w += 32) d = __dp4a(word_of(tok, w), mean[w], d);
            d = warp_sum(d);
            if (lane == 0) score[c] = d;
        }
        __syncthreads();
        if (tid == 0) {
            int best = 0;
            unsigned long long bd = (unsigned long long)score[0] * score[0];
            unsigned bn = nrm[rem[0]];
            for (int c = 1; c < n_rem; c++) {
                const unsigned long long d2 = (unsigned long long)score[c] * score[c];
                const unsigned n = nrm[rem[c]];
                // d2/n > bd/bn  (a zero vector has cosine 0)
                const bool gt = (n == 0) ? false : (bn == 0 ? d2 > 0 : d2 * bn > bd * n);
                if (gt) { best = c; bd = d2; bn = n; }
            }
            pick_s = best;
        }
        __syncthreads();
        take(pick_s, true);
        for (int t = 1; t < a.pack_len && n_rem > 0; t++) {
            for (int c = wic; c < n_rem; c += 8) {
                const int tok = rem[c];
                unsigned bits = 0;
                for (int w = lane; w < words; w += 32) bits += bitlen_sum4(mx[w], mn[w], word_of(tok, w));
                bits = warp_sum(bits);
                if (lane == 0) score[c] = bits;
            }
            __syncthreads();
            if (tid == 0) {
                int best = 0;
                for (int c = 1; c < n_rem; c++)
                    if (score[c] < score[best]) best = c;
                pick_s = best;
            }
            __syncthreads();
            take(pick_s, false);
        }
    }
    if (tid < a.block) a.order[((int64_t)b * (a.tokens / a.block) + blk) * a.block + tid] = out[tid];
}

int launch_greedy_order(const uint8_t* k_codes, const uint8_t* v_codes, int64_t seq_stride, uint8_t* order, int batch, int heads,
                        int tokens, int block, int pack_len, cudaStream_t st) {
    if (batch < 0 || heads <= 0 || tokens < 0 || block <= 0 || block > 128 || tokens % block || pack_len <= 0 || block % pack_len) return kBadArgument;
    if ((int64_t)batch * tokens == 0) return kOk;
    if (!k_codes || !v_codes || !order || (reinterpret_cast<uintptr_t>(k_codes) & 3) || (reinterpret_cast<uintptr_t>(v_codes) & 3) || (seq_stride & 3)) return kBadArgument;
    GreedyArgs a{k_codes, v_codes, seq_stride, order, tokens, block, pack_len, heads * 128};
    const int words = a.hidden / 2;
    const int smem = words * 12 + words * 8 + 128 * 8;
    if (smem > 200 * 1024) return kUnsupported;
    if (cudaFuncSetAttribute(greedy_order_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kCudaError;
    greedy_order_kernel<<<dim3(tokens / block, batch), 256, smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

// -------------------------------------------------------------------------------- size model
// The reference's bit_pack estimate (utils/compute.py:272-297) for one code tensor: packs of
// pack_len consecutive tokens of one feature; returns the sum over packs of bit_length(max - min)
// and the set of code values that occur (a 256-bit map), from which the host forms
//   bytes = (sum * pack_len + n_packs * (b + ceil(log2(b + 1)))) / 8,  b = ceil(log2(#values)).
__global__ void __launch_bounds__(256) size_model_kernel(const uint8_t* codes, int64_t seq_stride, int tokens, int hidden, int pack_len,
                                                         unsigned long long* bits_sum, unsigned* present) {
    const int p = blockIdx.x, b = blockIdx.y;
    const uint8_t* base = codes + (int64_t)b * seq_stride + (int64_t)p * pack_len * hidden;
    unsigned local = 0;
    unsigned seen[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int w = threadIdx.x; w < hidden / 4; w += 256) {
        unsigned lo[4] = {255, 255, 255, 255}, hi[4] = {0, 0, 0, 0};
        for (int t = 0; t < pack_len; t++) {
            const unsigned x = __ldg(reinterpret_cast<const unsigned*>(base + (int64_t)t * hidden) + w);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const unsigned c = (x >> (8 * k)) & 0xFFu;
                lo[k] = min(lo[k], c); hi[k] = max(hi[k], c);
#pragma unroll
                for (int i = 0; i < 8; i++) seen[i] |= (c >> 5) == (unsigned)i ? 1u << (c & 31u) : 0u;
            }
        }
#pragma unroll
        for (int k = 0; k < 4; k++) local += 32 - __clz(hi[k] - lo[k]);
    }
    local = warp_sum(local);
#pragma unroll
    for (int i = 0; i < 8; i++) seen[i] = __reduce_or_sync(0xffffffffu, seen[i]);
    if (lane_id() == 0) {
        atomicAdd(bits_sum, (unsigned long long)local);
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (seen[i]) atomicOr(present + i, seen[i]);
    }
}

int launch_size_model(const uint8_t* codes, int64_t seq_stride, int batch, int tokens, int hidden, int pack_len,
                      unsigned long long* bits_sum, unsigned* present, cudaStream_t st) {
    if (batch < 0 || tokens < 0 || hidden <= 0 || hidden % 4 || pack_len <= 0 || tokens % pack_len) return kBadArgument;
    if (!bits_sum || !present) return kBadArgument;
    if ((int64_t)batch * tokens == 0) return kOk;
    if (!codes || (reinterpret_cast<uintptr_t>(codes) & 3) || (seq_stride & 3)) return kBadArgument;
    size_model_kernel<<<dim3(tokens / pack_len, batch), 256, 0, st>>>(codes, seq_stride, tokens, hidden, pack_len, bits_sum, present);
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
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
