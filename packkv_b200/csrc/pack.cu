// Bit-pack encoder and decoder for uint8 code matrices (the reference's CPU codec,
// packkv_cuda_ext/src/{k,v}_{encode,decode}_cpu.cpp, done on the GPU).
//
// Work split: one warp owns one block (K: cb tokens x 128 channels, V: cb tokens x 64
// channels).  Encoding is three launches with no device-side waiting:
//   sizes  : every warp computes its block's byte size into block_info[blk][1]
//   scan   : one CTA per sequence turns sizes into byte offsets (block_info[blk][0]) and
//            updates the sequence's running stream length
//   write  : every warp rebuilds its block in shared memory (at the same 16-byte phase as
//            its destination) and copies it out with 16-byte stores
// HBM traffic per code: 2 bytes read (codes are read twice) + the stream bytes written.
#include "common.cuh"
#include "launch.h"
#include "pack_dev.cuh"

namespace pkv {


// Copies `size` bytes (plus up to 16 bytes of slack on either side, inside the stream
// allocation) from global `src` into shared memory so that the shared copy of src[0] has
// the same address modulo 16.  Returns the shared pointer that mirrors src.
__device__ __forceinline__ const uint8_t* warp_copy_in(uint8_t* sbuf16, const uint8_t* src, int size, int lane,
                                                       const uint8_t* lo, const uint8_t* hi) {
    int phase = (int)(reinterpret_cast<uintptr_t>(src) & 15);
    const uint8_t* a = src - phase;                 // 16-byte aligned start
    int total = (phase + size + 15) & ~15;
    for (int i = 16 * lane; i < total; i += 16 * 32) {
        const uint8_t* p = a + i;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (p >= lo && p + 16 <= hi) {
            v = *reinterpret_cast<const uint4*>(p);
        } else {                                    // ragged edge of the allocation
            unsigned q[4] = {0, 0, 0, 0};
#pragma unroll
            for (int b = 0; b < 16; b++)
                if (p + b >= lo && p + b < hi) q[b >> 2] |= (unsigned)p[b] << (8 * (b & 3));
            v = make_uint4(q[0], q[1], q[2], q[3]);
        }
        *reinterpret_cast<uint4*>(sbuf16 + i) = v;
    }
    return sbuf16 + phase;
}

struct PackParams {
    const uint8_t* codes;      // sequence s at codes + s*codes_seq_stride; (ctx_new, hidden) row-major
    int64_t codes_seq_stride;
    uint8_t* stream;           // sequence s at stream + s*stream_seq_stride
    int64_t stream_seq_stride;
    int64_t capacity;          // usable bytes per sequence stream
    uint32_t* info;            // sequence s at info + s*info_seq_stride*2
    int64_t info_seq_stride;   // in blocks
    uint32_t* stream_bytes;    // per sequence running length (in/out)
    unsigned* flags;
    int n_seq, nctx, nhid, hidden, cb, first_cb;
};

// =========================================================================================
// K
// =========================================================================================

template <int BITS>
__global__ void __launch_bounds__(kWarpsPerCta * 32) k_sizes_kernel(PackParams p) {
    const int lane = lane_id();
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t per_seq = (int64_t)p.nctx * p.nhid;
    if (warp >= per_seq * p.n_seq) return;
    const int s = (int)(warp / per_seq);
    const int rem = (int)(warp % per_seq);
    const int cbi = rem / p.nhid, hbi = rem % p.nhid;
    const KGeom g(p.cb, BITS);
    const uint8_t* base = p.codes + s * p.codes_seq_stride + (int64_t)cbi * p.cb * p.hidden + hbi * 128 + 4 * lane;
    unsigned lens = 0, over = 0;
    for (int r = 0; r < g.rounds; r++) {
        unsigned mn = 0xFFFFFFFFu, mx = 0;
#pragma unroll
        for (int t = 0; t < 16; t++) {
            unsigned u = __ldg(reinterpret_cast<const unsigned*>(base + (int64_t)(r * 16 + t) * p.hidden));
            mn = __vminu4(mn, u);
            mx = __vmaxu4(mx, u);
        }
        lens += sum_bitlen4(__vsub4(mx, mn));
        over |= mx & (0xFFFFFFFFu ^ (0x01010101u * ((1u << BITS) - 1u)));
    }
    lens = warp_sum(lens);
    over = __any_sync(0xffffffffu, over != 0);
    if (lane == 0) {
        p.info[(s * p.info_seq_stride + (int64_t)(p.first_cb + cbi) * p.nhid + hbi) * 2 + 1] =
            g.head_bytes + g.rounds * (g.min_bytes + g.len_bytes) + 2 * lens;
        if (over) atomicOr(p.flags, kFlagCodeRange);
    }
}

// One CTA per sequence: exclusive scan of the new blocks' sizes.
__global__ void __launch_bounds__(1024) scan_sizes_kernel(PackParams p) {
    __shared__ unsigned warp_tot[32];
    __shared__ unsigned carry_s;
    const int s = blockIdx.x;
    const int n = p.nctx * p.nhid;
    uint32_t* info = p.info + (s * p.info_seq_stride + (int64_t)p.first_cb * p.nhid) * 2;
    if (threadIdx.x == 0) carry_s = p.first_cb == 0 ? 0u : p.stream_bytes[s];
    __syncthreads();
    const int lane = lane_id(), w = threadIdx.x >> 5;
    for (int start = 0; start < n; start += 1024) {
        int i = start + threadIdx.x;
        const unsigned carry = carry_s;   // stable: last written before the previous barrier
        unsigned v = i < n ? info[2 * i + 1] : 0u;
        unsigned inc = warp_inclusive_sum(v);
        if (lane == 31) warp_tot[w] = inc;
        __syncthreads();
        if (w == 0) {
            unsigned t = warp_tot[lane];
            unsigned ti = warp_inclusive_sum(t);
            warp_tot[lane] = ti - t;   // exclusive prefix of warp totals
            if (lane == 31) carry_s = carry + ti;
        }
        __syncthreads();
        if (i < n) info[2 * i] = carry + warp_tot[w] + inc - v;
        __syncthreads();
    }
    if (threadIdx.x == 0) p.stream_bytes[s] = carry_s;
}

template <int BITS>
__global__ void __launch_bounds__(kWarpsPerCta * 32) k_write_kernel(PackParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int LB = len_field_bits(BITS);
    const int lane = lane_id();
    const int wic = threadIdx.x >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + wic;
    const int64_t per_seq = (int64_t)p.nctx * p.nhid;
    if (warp >= per_seq * p.n_seq) return;
    const int s = (int)(warp / per_seq);
    const int rem = (int)(warp % per_seq);
    const int cbi = rem / p.nhid, hbi = rem % p.nhid;
    const KGeom g(p.cb, BITS);
    const int slot = (g.head_bytes + g.rounds * (g.min_bytes + g.len_bytes + 128 * 2 * BITS) + 16 + 15) & ~15;
    const uint32_t* bi = p.info + (s * p.info_seq_stride + (int64_t)(p.first_cb + cbi) * p.nhid + hbi) * 2;
    const unsigned off = bi[0], size = bi[1];
    if ((int64_t)off + size > p.capacity) {
        if (lane == 0) atomicOr(p.flags, kFlagStreamOverflow);
        return;
    }
    uint8_t* dst = p.stream + s * p.stream_seq_stride + off;
    uint8_t* stage = smem + wic * slot + (reinterpret_cast<uintptr_t>(dst) & 15);
    const uint8_t* base = p.codes + s * p.codes_seq_stride + (int64_t)cbi * p.cb * p.hidden + hbi * 128 + 4 * lane;

    int pos = g.head_bytes;
    unsigned round_end = 0;
    for (int r = 0; r < g.rounds; r++) {
        unsigned u[16];
        unsigned mn = 0xFFFFFFFFu, mx = 0;
#pragma unroll
        for (int t = 0; t < 16; t++) {
            u[t] = __ldg(reinterpret_cast<const unsigned*>(base + (int64_t)(r * 16 + t) * p.hidden));
            mn = __vminu4(mn, u[t]);
            mx = __vmaxu4(mx, u[t]);
        }
        const unsigned d = __vsub4(mx, mn);
        unsigned minword = 0, lenword = 0, lens4 = 0;
        int len[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            len[j] = bit_length_u32((d >> (8 * j)) & 0xFFu);
            minword |= (((mn >> (8 * j)) & 0xFFu) & ((1u << BITS) - 1u)) << (j * BITS);
            lenword |= (unsigned)len[j] << (j * LB);
            lens4 |= (unsigned)len[j] << (8 * j);
        }
        store_lane_fields(stage + pos, lane, 4 * BITS, minword);
        store_lane_fields(stage + pos + g.min_bytes, lane, 4 * LB, lenword);
        // byte offsets of this lane's four packs: packs are ordered j-major, lane-minor
        const unsigned inc = warp_inclusive_sum(lens4);
        const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
        const unsigned exc = inc - lens4;
        uint8_t* packs = stage + pos + g.min_bytes + g.len_bytes;
        unsigned before = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint64_t w = 0;
            const unsigned m = (mn >> (8 * j)) & 0xFFu;
#pragma unroll
            for (int t = 0; t < 16; t++) w = (w << len[j]) | (uint64_t)(((u[t] >> (8 * j)) & 0xFFu) - m);
            store_pack_smem(packs + 2 * (before + ((exc >> (8 * j)) & 0xFFu)), w, len[j]);
            before += (tot >> (8 * j)) & 0xFFu;
        }
        const unsigned round_size = g.min_bytes + g.len_bytes + 2 * before;
        round_end += round_size;
        if (lane == 0) *reinterpret_cast<uint16_t*>(stage + 2 * r) = (uint16_t)round_end;
        pos += round_size;
    }
    __syncwarp();
    warp_copy_out(dst, stage, (int)size, lane);
}

template <int BITS>
__global__ void __launch_bounds__(kWarpsPerCta * 32) k_decode_kernel(PackParams p, int64_t stream_len_cap) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int LB = len_field_bits(BITS);
    const int lane = lane_id();
    const int wic = threadIdx.x >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + wic;
    const int64_t per_seq = (int64_t)p.nctx * p.nhid;
    if (warp >= per_seq * p.n_seq) return;
    const int s = (int)(warp / per_seq);
    const int rem = (int)(warp % per_seq);
    const int cbi = rem / p.nhid, hbi = rem % p.nhid;
    const KGeom g(p.cb, BITS);
    const int bound = g.head_bytes + g.rounds * (g.min_bytes + g.len_bytes + 128 * 2 * BITS);
    const int slot = (bound + 48 + 15) & ~15;
    const uint32_t* bi = p.info + (s * p.info_seq_stride + (int64_t)(p.first_cb + cbi) * p.nhid + hbi) * 2;
    const unsigned off = bi[0], size = bi[1];
    if ((int64_t)off + size > stream_len_cap || (int)size > bound || (int)size < g.head_bytes) {
        if (lane == 0) atomicOr(p.flags, kFlagBadStream);
        return;
    }
    const uint8_t* sbase = p.stream + s * p.stream_seq_stride;
    const uint8_t* blk = warp_copy_in(smem + wic * slot, sbase + off, (int)size, lane, sbase, sbase + stream_len_cap);
    __syncwarp();
    uint8_t* out = const_cast<uint8_t*>(p.codes) + s * p.codes_seq_stride + (int64_t)cbi * p.cb * p.hidden + hbi * 128 + 4 * lane;
    int pos = g.head_bytes;
    bool bad = false;
    for (int r = 0; r < g.rounds; r++) {
        if (pos + g.min_bytes + g.len_bytes > (int)size) { bad = true; break; }
        const unsigned minword = load_lane_field(blk + pos, lane, 4 * BITS);
        const unsigned lenword = load_lane_field(blk + pos + g.min_bytes, lane, 4 * LB);
        unsigned lens4 = 0;
        int len[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            len[j] = (lenword >> (j * LB)) & ((1u << LB) - 1u);
            if (len[j] > BITS) { len[j] = BITS; bad = true; }
            lens4 |= (unsigned)len[j] << (8 * j);
        }
        const unsigned inc = warp_inclusive_sum(lens4);
        const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
        const unsigned exc = inc - lens4;
        const uint8_t* packs = blk + pos + g.min_bytes + g.len_bytes;
        unsigned before = 0;
        unsigned u[16];
#pragma unroll
        for (int t = 0; t < 16; t++) u[t] = 0;
        const unsigned total_words = (tot & 0xFF) + ((tot >> 8) & 0xFF) + ((tot >> 16) & 0xFF) + (tot >> 24);
        const bool fits = pos + g.min_bytes + g.len_bytes + 2 * (int)total_words <= (int)size;
        if (!fits) { bad = true; break; }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint64_t w = load_u64_align2(packs + 2 * (before + ((exc >> (8 * j)) & 0xFFu)));
            const unsigned m = (minword >> (j * BITS)) & ((1u << BITS) - 1u);
            const unsigned mask = (1u << len[j]) - 1u;
#pragma unroll
            for (int t = 0; t < 16; t++) {
                unsigned c = ((unsigned)(w >> (len[j] * (15 - t))) & mask) + m;
                u[t] |= (c & 0xFFu) << (8 * j);
            }
            before += (tot >> (8 * j)) & 0xFFu;
        }
#pragma unroll
        for (int t = 0; t < 16; t++)
            *reinterpret_cast<unsigned*>(out + (int64_t)(r * 16 + t) * p.hidden) = u[t];
        pos += g.min_bytes + g.len_bytes + 2 * before;
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(p.flags, kFlagBadStream);
}

// =========================================================================================
// V
// =========================================================================================

// loads the cb x 64 code tile of one V block into shared memory (row-major, 64 B rows)
__device__ __forceinline__ void v_load_tile(uint8_t* tile, const uint8_t* src, int cb, int hidden, int lane) {
    // 4 lanes per row (16 B each), 8 rows per step
    const int sub = lane & 3, row0 = lane >> 2;
    for (int r = row0; r < cb; r += 8) {
        uint4 v = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)r * hidden + 16 * sub));
        *reinterpret_cast<uint4*>(tile + r * 64 + 16 * sub) = v;
    }
}

template <int BITS>
__global__ void __launch_bounds__(kWarpsPerCta * 32) v_sizes_kernel(PackParams p) {
    const int lane = lane_id();
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    const int64_t per_seq = (int64_t)p.nctx * p.nhid;
    if (warp >= per_seq * p.n_seq) return;
    const int s = (int)(warp / per_seq);
    const int rem = (int)(warp % per_seq);
    const int cbi = rem / p.nhid, hbi = rem % p.nhid;
    const VGeom g(p.cb, BITS);
    // lane owns channel pair (2*lane, 2*lane+1): u16 loads keep rows coalesced (64 B per row)
    const uint8_t* base = p.codes + s * p.codes_seq_stride + (int64_t)cbi * p.cb * p.hidden + hbi * 64 + 2 * lane;
    unsigned lens = 0, over = 0;
    for (int pk = 0; pk < p.cb / 16; pk++) {
        unsigned mn = 0xFFFFu, mx = 0;
#pragma unroll
        for (int t = 0; t < 16; t++) {
            unsigned u = __ldg(reinterpret_cast<const uint16_t*>(base + (int64_t)(pk * 16 + t) * p.hidden));
            mn = __vminu4(mn, u);
            mx = __vmaxu4(mx, u);
        }
        lens += sum_bitlen4(__vsub4(mx, mn));
        over |= mx & (0xFFFFu ^ (0x0101u * ((1u << BITS) - 1u)));
    }
    lens = warp_sum(lens);
    over = __any_sync(0xffffffffu, over != 0);
    if (lane == 0) {
        p.info[(s * p.info_seq_stride + (int64_t)(p.first_cb + cbi) * p.nhid + hbi) * 2 + 1] =
            g.head_bytes + g.nseg * (g.min_bytes + g.len_bytes) + 2 * lens;
        if (over) atomicOr(p.flags, kFlagCodeRange);
    }
}

template <int BITS>
__global__ void __launch_bounds__(kWarpsPerCta * 32) v_write_kernel(PackParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int LB = len_field_bits(BITS);
    const int lane = lane_id();
    const int wic = threadIdx.x >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + wic;
    const int64_t per_seq = (int64_t)p.nctx * p.nhid;
    if (warp >= per_seq * p.n_seq) return;
    const int s = (int)(warp / per_seq);
    const int rem = (int)(warp % per_seq);
    const int cbi = rem / p.nhid, hbi = rem % p.nhid;
    const VGeom g(p.cb, BITS);
    const int bound = g.head_bytes + g.nseg * (g.min_bytes + g.len_bytes + 32 * g.ppt * 2 * BITS);
    const int slot = ((bound + 16 + 15) & ~15) + p.cb * 64;
    const uint32_t* bi = p.info + (s * p.info_seq_stride + (int64_t)(p.first_cb + cbi) * p.nhid + hbi) * 2;
    const unsigned off = bi[0], size = bi[1];
    if ((int64_t)off + size > p.capacity) {
        if (lane == 0) atomicOr(p.flags, kFlagStreamOverflow);
        return;
    }
    uint8_t* tile = smem + wic * slot;
    uint8_t* dst = p.stream + s * p.stream_seq_stride + off;
    uint8_t* stage = tile + p.cb * 64 + (reinterpret_cast<uintptr_t>(dst) & 15);
    v_load_tile(tile, p.codes + s * p.codes_seq_stride + (int64_t)cbi * p.cb * p.hidden + hbi * 64, p.cb, p.hidden, lane);
    __syncwarp();

    int pos = g.head_bytes;
    unsigned seg_end = 0;
    for (int w = 0; w < 2; w++)
        for (int r = 0; r < g.rpw; r++) {
            const uint8_t* col = tile + (r * g.ppt * 16) * 64 + w * 32 + lane;
            unsigned minword = 0, lenword = 0, lens4 = 0;
            uint64_t wd[4];
            int len[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                len[q] = 0;
                wd[q] = 0;
                if (q < g.ppt) {
                    unsigned c[16];
                    unsigned mn = 255, mx = 0;
#pragma unroll
                    for (int t = 0; t < 16; t++) {
                        c[t] = col[(q * 16 + t) * 64];
                        mn = min(mn, c[t]);
                        mx = max(mx, c[t]);
                    }
                    len[q] = bit_length_u32(mx - mn);
#pragma unroll
                    for (int t = 0; t < 16; t++) wd[q] = (wd[q] << len[q]) | (uint64_t)(c[t] - mn);
                    minword |= (mn & ((1u << BITS) - 1u)) << (q * BITS);
                    lenword |= (unsigned)len[q] << (q * LB);
                    lens4 |= (unsigned)len[q] << (8 * q);
                }
            }
            store_lane_fields(stage + pos, lane, g.ppt * BITS, minword);
            store_lane_fields(stage + pos + g.min_bytes, lane, g.ppt * LB, lenword);
            const unsigned inc = warp_inclusive_sum(lens4);
            const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
            const unsigned exc = inc - lens4;
            uint8_t* packs = stage + pos + g.min_bytes + g.len_bytes;
            unsigned before = 0;
#pragma unroll
            for (int q = 0; q < 4; q++)
                if (q < g.ppt) {
                    store_pack_smem(packs + 2 * (before + ((exc >> (8 * q)) & 0xFFu)), wd[q], len[q]);
                    before += (tot >> (8 * q)) & 0xFFu;
                }
            const unsigned seg_size = g.min_bytes + g.len_bytes + 2 * before;
            seg_end += seg_size;
            if (lane == 0) *reinterpret_cast<uint16_t*>(stage + 2 * (w * g.rpw + r)) = (uint16_t)seg_end;
            pos += seg_size;
        }
    __syncwarp();
    warp_copy_out(dst, stage, (int)size, lane);
}

template <int BITS>
__global__ void __launch_bounds__(kWarpsPerCta * 32) v_decode_kernel(PackParams p, int64_t stream_len_cap) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int LB = len_field_bits(BITS);
    const int lane = lane_id();
    const int wic = threadIdx.x >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + wic;
    const int64_t per_seq = (int64_t)p.nctx * p.nhid;
    if (warp >= per_seq * p.n_seq) return;
    const int s = (int)(warp / per_seq);
    const int rem = (int)(warp % per_seq);
    const int cbi = rem / p.nhid, hbi = rem % p.nhid;
    const VGeom g(p.cb, BITS);
    const int bound = g.head_bytes + g.nseg * (g.min_bytes + g.len_bytes + 32 * g.ppt * 2 * BITS);
    const int slot = ((bound + 48 + 15) & ~15) + p.cb * 64;
    const uint32_t* bi = p.info + (s * p.info_seq_stride + (int64_t)(p.first_cb + cbi) * p.nhid + hbi) * 2;
    const unsigned off = bi[0], size = bi[1];
    if ((int64_t)off + size > stream_len_cap || (int)size > bound || (int)size < g.head_bytes) {
        if (lane == 0) atomicOr(p.flags, kFlagBadStream);
        return;
    }
    uint8_t* tile = smem + wic * slot;
    const uint8_t* sbase = p.stream + s * p.stream_seq_stride;
    const uint8_t* blk = warp_copy_in(tile + p.cb * 64, sbase + off, (int)size, lane, sbase, sbase + stream_len_cap);
    __syncwarp();
    int pos = g.head_bytes;
    bool bad = false;
    for (int w = 0; w < 2 && !bad; w++)
        for (int r = 0; r < g.rpw; r++) {
            if (pos + g.min_bytes + g.len_bytes > (int)size) { bad = true; break; }
            const unsigned minword = load_lane_field(blk + pos, lane, g.ppt * BITS);
            const unsigned lenword = load_lane_field(blk + pos + g.min_bytes, lane, g.ppt * LB);
            unsigned lens4 = 0;
            int len[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                len[q] = q < g.ppt ? (int)((lenword >> (q * LB)) & ((1u << LB) - 1u)) : 0;
                if (len[q] > BITS) { len[q] = BITS; bad = true; }
                lens4 |= (unsigned)len[q] << (8 * q);
            }
            const unsigned inc = warp_inclusive_sum(lens4);
            const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
            const unsigned exc = inc - lens4;
            const unsigned total_words = (tot & 0xFF) + ((tot >> 8) & 0xFF) + ((tot >> 16) & 0xFF) + (tot >> 24);
            if (pos + g.min_bytes + g.len_bytes + 2 * (int)total_words > (int)size) { bad = true; break; }
            const uint8_t* packs = blk + pos + g.min_bytes + g.len_bytes;
            uint8_t* col = tile + (r * g.ppt * 16) * 64 + w * 32 + lane;
            unsigned before = 0;
#pragma unroll
            for (int q = 0; q < 4; q++)
                if (q < g.ppt) {
                    const uint64_t wd = load_u64_align2(packs + 2 * (before + ((exc >> (8 * q)) & 0xFFu)));
                    const unsigned m = (minword >> (q * BITS)) & ((1u << BITS) - 1u);
                    const unsigned mask = (1u << len[q]) - 1u;
#pragma unroll
                    for (int t = 0; t < 16; t++)
                        col[(q * 16 + t) * 64] = (uint8_t)(((unsigned)(wd >> (len[q] * (15 - t))) & mask) + m);
                    before += (tot >> (8 * q)) & 0xFFu;
                }
            pos += g.min_bytes + g.len_bytes + 2 * before;
        }
    __syncwarp();
    if (__any_sync(0xffffffffu, bad)) {
        if (lane == 0) atomicOr(p.flags, kFlagBadStream);
        return;
    }
    uint8_t* out = const_cast<uint8_t*>(p.codes) + s * p.codes_seq_stride + (int64_t)cbi * p.cb * p.hidden + hbi * 64;
    const int sub = lane & 3, row0 = lane >> 2;
    for (int r = row0; r < p.cb; r += 8)
        *reinterpret_cast<uint4*>(out + (int64_t)r * p.hidden + 16 * sub) = *reinterpret_cast<const uint4*>(tile + r * 64 + 16 * sub);
}

// =========================================================================================
// host launchers
// =========================================================================================

static inline int k_slot_bytes(int cb, int bits, int extra) {
    KGeom g(cb, bits);
    return (g.head_bytes + g.rounds * (g.min_bytes + g.len_bytes + 128 * 2 * bits) + extra + 15) & ~15;
}
static inline int v_slot_bytes(int cb, int bits, int extra) {
    VGeom g(cb, bits);
    return ((g.head_bytes + g.nseg * (g.min_bytes + g.len_bytes + 32 * g.ppt * 2 * bits) + extra + 15) & ~15) + cb * 64;
}

template <typename K>
static int set_smem(K kernel, int bytes) {
    if (bytes > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return kCudaError;
    }
    return kOk;
}

#define PKV_DISPATCH_BITS(bits, ...) \
    switch (bits) {                   \
        case 2: { constexpr int B = 2; __VA_ARGS__; break; } \
        case 3: { constexpr int B = 3; __VA_ARGS__; break; } \
        case 4: { constexpr int B = 4; __VA_ARGS__; break; } \
        default: return kUnsupported; \
    }

static bool geometry_ok(bool is_k, const CodecShape& sh) {
    if (sh.bits < 2 || sh.bits > 4) return false;
    if (is_k) {
        if (sh.hb != 128 || (sh.cb != 32 && sh.cb != 64 && sh.cb != 128)) return false;
    } else {
        if (sh.hb != 64 || (sh.cb != 32 && sh.cb != 64 && sh.cb != 128)) return false;
    }
    if (sh.n_seq < 0 || sh.ctx_len < 0 || sh.hidden <= 0 || sh.ctx_len % sh.cb || sh.hidden % sh.hb) return false;
    if (sh.first_cb < 0) return false;
    return true;
}

static PackParams make_params(const CodecShape& sh, const CodecBuffers& b) {
    PackParams p;
    p.codes = b.codes; p.codes_seq_stride = b.codes_seq_stride;
    p.stream = b.stream; p.stream_seq_stride = b.stream_seq_stride; p.capacity = b.capacity;
    p.info = b.info; p.info_seq_stride = b.info_seq_stride;
    p.stream_bytes = b.stream_bytes; p.flags = b.flags;
    p.n_seq = sh.n_seq; p.nctx = sh.ctx_len / sh.cb; p.nhid = sh.hidden / sh.hb;
    p.hidden = sh.hidden; p.cb = sh.cb; p.first_cb = sh.first_cb;
    return p;
}

int launch_scan_sizes(const CodecShape& sh, const CodecBuffers& b, cudaStream_t st) {
    PackParams p = make_params(sh, b);
    if (p.n_seq <= 0) return kOk;
    scan_sizes_kernel<<<p.n_seq, 1024, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

int launch_encode(bool is_k, const CodecShape& sh, const CodecBuffers& b, cudaStream_t st) {
    if (!geometry_ok(is_k, sh)) return (sh.bits < 2 || sh.bits > 4 || (sh.cb != 32 && sh.cb != 64 && sh.cb != 128)) ? kUnsupported : kBadArgument;
    if ((int64_t)(sh.ctx_len / sh.cb) * (sh.hidden / sh.hb) * sh.n_seq == 0) return kOk;   // nothing to do
    if (!b.codes || !b.stream || !b.info || !b.stream_bytes || !b.flags) return kBadArgument;
    if ((reinterpret_cast<uintptr_t>(b.codes) & 15) || (b.codes_seq_stride & 15) || (reinterpret_cast<uintptr_t>(b.stream) & 1) ||
        (b.stream_seq_stride & 1))
        return kBadArgument;
    PackParams p = make_params(sh, b);
    const int64_t nwarps = (int64_t)p.nctx * p.nhid * p.n_seq;
    if (nwarps == 0) return kOk;
    const unsigned grid = (unsigned)((nwarps + kWarpsPerCta - 1) / kWarpsPerCta);
    const int threads = kWarpsPerCta * 32;
    if (is_k) {
        PKV_DISPATCH_BITS(sh.bits, (k_sizes_kernel<B><<<grid, threads, 0, st>>>(p)));
    } else {
        PKV_DISPATCH_BITS(sh.bits, (v_sizes_kernel<B><<<grid, threads, 0, st>>>(p)));
    }
    scan_sizes_kernel<<<p.n_seq, 1024, 0, st>>>(p);
    if (is_k) {
        const int smem = kWarpsPerCta * k_slot_bytes(sh.cb, sh.bits, 16);
        PKV_DISPATCH_BITS(sh.bits, { if (set_smem(k_write_kernel<B>, smem)) return kCudaError;
                                     k_write_kernel<B><<<grid, threads, smem, st>>>(p); });
    } else {
        const int smem = kWarpsPerCta * v_slot_bytes(sh.cb, sh.bits, 16);
        PKV_DISPATCH_BITS(sh.bits, { if (set_smem(v_write_kernel<B>, smem)) return kCudaError;
                                     v_write_kernel<B><<<grid, threads, smem, st>>>(p); });
    }
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

int launch_decode(bool is_k, const CodecShape& sh, const CodecBuffers& b, cudaStream_t st) {
    if (!geometry_ok(is_k, sh)) return (sh.bits < 2 || sh.bits > 4 || (sh.cb != 32 && sh.cb != 64 && sh.cb != 128)) ? kUnsupported : kBadArgument;
    if ((int64_t)(sh.ctx_len / sh.cb) * (sh.hidden / sh.hb) * sh.n_seq == 0) return kOk;
    if (!b.codes || !b.stream || !b.info || !b.flags) return kBadArgument;
    if ((reinterpret_cast<uintptr_t>(b.codes) & 15) || (b.codes_seq_stride & 15) || (reinterpret_cast<uintptr_t>(b.stream) & 1) ||
        (b.stream_seq_stride & 1))
        return kBadArgument;
    PackParams p = make_params(sh, b);
    const int64_t nwarps = (int64_t)p.nctx * p.nhid * p.n_seq;
    if (nwarps == 0) return kOk;
    const unsigned grid = (unsigned)((nwarps + kWarpsPerCta - 1) / kWarpsPerCta);
    const int threads = kWarpsPerCta * 32;
    if (is_k) {
        const int smem = kWarpsPerCta * k_slot_bytes(sh.cb, sh.bits, 48);
        PKV_DISPATCH_BITS(sh.bits, { if (set_smem(k_decode_kernel<B>, smem)) return kCudaError;
                                     k_decode_kernel<B><<<grid, threads, smem, st>>>(p, b.capacity); });
    } else {
        const int smem = kWarpsPerCta * v_slot_bytes(sh.cb, sh.bits, 48);
        PKV_DISPATCH_BITS(sh.bits, { if (set_smem(v_decode_kernel<B>, smem)) return kCudaError;
                                     v_decode_kernel<B><<<grid, threads, smem, st>>>(p, b.capacity); });
    }
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

}  // namespace pkv
