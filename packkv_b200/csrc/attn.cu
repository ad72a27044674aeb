// Fused decompress-attention decode for one query token per sequence.
//
// Replaces, in one launch over the packed streams, the reference's kq_mat_vec_mul + fused_kq
// (packkv_cuda_ext/src/kernels.cu:426-535, fused_kernels.cu:13-76), torch softmax
// (evaluation/evaluation.py:1040-1049), wv_mat_vec_mul + fused_wv (kernels.cu:632-765,
// fused_kernels.cu:187-261) and, for numerics, the model path's dequantise-then-attend
// (models/cache/packkv_quant.py:45-85 + models/llama.py:177-212).  Decompressed K/V never go
// to HBM, and in the single launch neither do scores or partial results (the two-launch form for
// launches whose pairs do not fill the GPU hands scores and per-cluster rows over through a scratch).
//
// Numerics follow the reference's rounding points so the result can be compared with its
// decompress-then-attend path: every K and V element is dequantised to the element type
// exactly as (code + zero) * scale (two roundings, utils/compute.py:178); scores are rounded
// to the element type after the dot product and again after * scaling (llama.py:200); the
// softmax runs in fp32 over ALL tokens and its probabilities are rounded to the element type
// before the second contraction (llama.py:208-210), which accumulates in fp32.
//
// Because the probabilities need the global max and sum before they can be rounded, the
// sequence is split over a thread-block CLUSTER instead of over independent CTAs with a later merge:
// grid = (cluster_size, kv_heads, batch), one cluster per (sequence, KV head).
//   phase 1  every warp of the cluster walks its token tiles: K blocks are staged in shared memory
//            by bulk copies (one instruction of one lane per block, completion on an mbarrier),
//            unpacked and dequantised by the lane that owns the channel, transposed through a
//            small shared-memory tile into mma fragments and contracted with q on the tensor cores;
//            scores stay in the warp's shared memory.
//   exchange per-CTA (max, sum) go through distributed shared memory, one cluster barrier.
//   phase 2  scores -> probabilities in place; V packs are fetched by the lane whose mma fragment
//            needs them (a pack is 16 tokens of one channel = one row segment of the A operand), so
//            V needs no transposition at all.
//   reduce   warps -> CTA in shared memory, CTAs -> rank 0 through distributed shared memory.
//
// Unpack, per pack (16 codes of `len` bits, token 0 in the top bits): one 8-byte window at a 2-byte
// aligned offset (warp scan of the lengths), then per 8 codes one shift-and-select that puts codes
// i and i+4 sixteen bits apart and four shift-mask-or steps that yield the element-type pairs
// (bias + code_i, bias + code_{i+4}) directly (the bias is the exponent pattern under which the
// code bits are the low mantissa bits).  The pairing (i, i+4) fixes a token order inside each group
// of 16, which the score / probability / parameter arrays in shared memory follow.
#include <cooperative_groups.h>
#include <cstdlib>
#include <type_traits>

#include "attn.cuh"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace pkv {

#ifndef PKV_ATTN_WARPS
#define PKV_ATTN_WARPS 4
#endif
constexpr int kAW = PKV_ATTN_WARPS;   // warps per CTA (1, 2 or 4)
#ifndef PKV_ATTN_CTAS
#define PKV_ATTN_CTAS (16 / PKV_ATTN_WARPS)
#endif
constexpr int kMaxCtasPerSm = PKV_ATTN_CTAS;  // register budget: 65536 / (128 * 4) -> 128 per thread, 96 for 5
constexpr int kD = 128;           // head dimension
constexpr int kSmCount = 148;
constexpr unsigned kWaitSpins = 1u << 22;   // bounded mbarrier wait (each try suspends for a while by itself)
#ifndef PKV_ATTN_CTAS_SCORES
#define PKV_ATTN_CTAS_SCORES PKV_ATTN_CTAS   // the two-launch form's kernels may take other register budgets
#endif
#ifndef PKV_ATTN_CTAS_VALUES
#define PKV_ATTN_CTAS_VALUES PKV_ATTN_CTAS
#endif
#ifndef PKV_ONE_CHAIN
#define PKV_ONE_CHAIN 0
#endif
#ifndef PKV_ABL
#define PKV_ABL 0
#endif

// ---- element-type traits --------------------------------------------------------------------
template <typename T> struct Tr;

template <> struct Tr<__half> {
    using T2 = __half2;
    static constexpr unsigned kMagic2 = 0x64006400u;  // 0x6400 | b == 1024 + b, exact
    static constexpr unsigned kMagicB = 0x64646464u;
    static constexpr float kBias = 1024.f;
    static __device__ __forceinline__ T2 bias2() { return __float2half2_rn(1024.f); }
    static __device__ __forceinline__ T2 zmax2() { return __float2half2_rn(2048.f - 16.f); }
    static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
    static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
    static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
    static __device__ __forceinline__ T2 dup(__half x) { return __half2half2(x); }
    static __device__ __forceinline__ float2 unpack2(unsigned v) { return __half22float2(*reinterpret_cast<const __half2*>(&v)); }
    static __device__ __forceinline__ unsigned pack2(float lo, float hi) { __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<unsigned*>(&h); }
    static __device__ __forceinline__ void mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

template <> struct Tr<__nv_bfloat16> {
    using T2 = __nv_bfloat162;
    static constexpr unsigned kMagic2 = 0x43004300u;  // 0x4300 | b == 128 + b, exact
    static constexpr unsigned kMagicB = 0x43434343u;
    static constexpr float kBias = 128.f;
    static __device__ __forceinline__ T2 bias2() { return __float2bfloat162_rn(128.f); }
    static __device__ __forceinline__ T2 zmax2() { return __float2bfloat162_rn(256.f - 16.f); }
    static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
    static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
    static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ T2 dup(__nv_bfloat16 x) { return __bfloat162bfloat162(x); }
    static __device__ __forceinline__ float2 unpack2(unsigned v) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v)); }
    static __device__ __forceinline__ unsigned pack2(float lo, float hi) { __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<unsigned*>(&h); }
    static __device__ __forceinline__ void mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

template <typename T2> __device__ __forceinline__ unsigned as_u(T2 v) { return *reinterpret_cast<unsigned*>(&v); }
template <typename T2> __device__ __forceinline__ T2 as_t2(unsigned v) { return *reinterpret_cast<T2*>(&v); }

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void cp_async16_zfill(unsigned smem_dst, const void* gsrc, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_dst), "l"(gsrc), "r"(valid ? 16 : 0));
}

// ---- mbarrier + bulk copy (global -> this CTA's shared memory, no multicast) ------------------
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// exp(x) for x <= 0 (softmax arguments): one multiply and one MUFU; results below the normal
// range flush to zero, which the rounding to the element type does anyway
__device__ __forceinline__ float fast_exp(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
    return y;
}
// four 8x8 b16 matrices, transposed on load: lane l passes the address of row l%8 of matrix l/8
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned addr, unsigned (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ uint2 lds64(unsigned a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ unsigned lds8(unsigned a) {
    unsigned v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void sts64(unsigned a, unsigned x, unsigned y) { asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a), "r"(x), "r"(y) : "memory"); }

// header fields of width w at bits 0, w, 2w, 3w of a lane word -> one byte each
struct FieldSpread { int s1, s2; unsigned m1, m2; };
__device__ __forceinline__ unsigned spread_fields(unsigned x, const FieldSpread& f) {
    const unsigned y = (x | (x << f.s1)) & f.m1;
    return (y | (y << f.s2)) & f.m2;
}
__host__ inline FieldSpread make_field_spread(int w) {
    return FieldSpread{16 - 2 * w, 8 - w, ((1u << (2 * w)) - 1u) * 0x00010001u, ((1u << w) - 1u) * 0x01010101u};
}
__device__ __forceinline__ unsigned byte_of(unsigned x, int j) { return __byte_perm(x, 0, 0x4440 + j); }

// Reads of data that nothing writes while it is being read (a staged stream block, the length table): no
// "memory" clobber and not volatile, so the compiler may schedule them across the exchange-tile traffic.  The
// address must be derived from a value defined after the wait that made the data visible.
__device__ __forceinline__ unsigned ldp32(unsigned a) { unsigned v; asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ unsigned ldp16(unsigned a) { unsigned short v; asm("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a)); return v; }
__device__ __forceinline__ unsigned ldp8(unsigned a) { unsigned v; asm("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
// 64-bit window at shared address a (2-byte aligned): three aligned 32-bit loads, two funnel shifts
__device__ __forceinline__ void ldp_u64_align2(unsigned a, unsigned& lo, unsigned& hi) {
    const unsigned wa = a & ~3u, sh = (a & 2u) * 8u;
    const unsigned w0 = ldp32(wa), w1 = ldp32(wa + 4), w2 = ldp32(wa + 8);
    lo = __funnelshift_r(w0, w1, sh);
    hi = __funnelshift_r(w1, w2, sh);
}
// lane word of W bits (8, 12 or 16) at bit lane * W of a header field that starts at a 2-byte aligned address
template <int W> __device__ __forceinline__ unsigned lane_word(unsigned hdr, int lane) {
    if (W == 16) return ldp16(hdr + 2 * lane);
    if (W == 8) return ldp8(hdr + lane);
    const unsigned ad = hdr + 2 * ((3 * lane) >> 2);
    const unsigned w = ldp16(ad) | (ldp16(ad + 2) << 16);
    return (w >> (4 * ((3 * lane) & 3))) & 0xFFFu;
}
// four fields of W bits at bits 0, W, 2W, 3W -> one byte each
template <int W> __device__ __forceinline__ unsigned spread_const(unsigned x) {
    constexpr unsigned m1 = ((1u << (2 * W)) - 1u) * 0x00010001u, m2 = ((1u << W) - 1u) * 0x01010101u;
    const unsigned y = (x | (x << (16 - 2 * W))) & m1;
    return (y | (y << (8 - W))) & m2;
}

// Eight codes of `len` bits (code 0 in the top bits of x, garbage above bit 8*len allowed) -> four
// registers of element-type pairs: r[k] = (bias + code_{7-k}, bias + code_{3-k}) as (low, high) halves.
// s1 = 16 - 4 len, m16 = (2^len - 1) * 0x00010001.
template <unsigned MAGIC>
__device__ __forceinline__ void unpack8(unsigned x, unsigned s1, unsigned len, unsigned m16, unsigned (&r)[4]) {
    // codes 4..7 stay in the low half, codes 0..3 move to the high half: code i and i+4 end up 16 bits apart
    unsigned y = ((x << s1) & 0xFFFF0000u) | (x & 0x0000FFFFu);
    r[0] = (y & m16) | MAGIC;
    y >>= len;
    r[1] = (y & m16) | MAGIC;
    y >>= len;
    r[2] = (y & m16) | MAGIC;
    y >>= len;
    r[3] = (y & m16) | MAGIC;
}
// Token held by the (low, high) halves of register k of the group of eight that starts at token 8*grp:
//   k:      0      1      2      3
//   pair: (7,3)  (6,2)  (5,1)  (4,0)
// The shared-memory arrays that are read as such pairs (V scales, zero-points, probabilities; token-mode K
// parameters) store, per group of 16 tokens, the words [(7,3) (6,2) (5,1) (4,0) (15,11) (14,10) (13,9) (12,8)].
// A lane that holds the natural-order words n_e = (2e, 2e+1) and n_{e+2} = (2e+4, 2e+5) of a group of eight
// (e = 0, 1) forms the two paired words it owns; they are adjacent: word index 2 - 2e and 3 - 2e.
__device__ __forceinline__ void pair_words(unsigned ne, unsigned ne2, unsigned& w_first, unsigned& w_second) {
    w_first = __byte_perm(ne, ne2, 0x3276);    // (2e+5, 2e+1): word 2 - 2e
    w_second = __byte_perm(ne, ne2, 0x1054);   // (2e+4, 2e):   word 3 - 2e
}

// q fragments for the residual (uncompressed) tiles.  mma step j = 2m + b covers, for the lanes with c = lane & 3,
// the channels 32m + 8c + {2b, 2b+4} (k = 2c, 2c+1) and 32m + 8c + {2b+1, 2b+5} (k = 2c+8, 2c+9).  From the 8
// consecutive elements x0..x7 of channels 32m + 8c.. this forms the operand registers of steps 2m and 2m+1:
// f[b][0] = (x[2b], x[2b+4]), f[b][1] = (x[2b+1], x[2b+5]).
__device__ __forceinline__ void pair_shuffle(const uint4& v, unsigned (&f0)[2], unsigned (&f1)[2]) {
    f0[0] = __byte_perm(v.x, v.z, 0x5410); f0[1] = __byte_perm(v.x, v.z, 0x7632);
    f1[0] = __byte_perm(v.y, v.w, 0x5410); f1[1] = __byte_perm(v.y, v.w, 0x7632);
}

struct AttnDev {
    AttnArgs a;
    int cluster;         // CTAs per (sequence, kv head)
    int tile;            // tokens per warp tile: 128 or 64
    int tiles_total;     // n_comp / tile
    int tpw;             // max tiles per warp
    int rtw;             // max residual tiles (16 tokens) per warp
    int rows;            // score rows kept per tile (q heads of the group, rounded up to even)
    int slot;            // bytes of one staging slot
    int nslots;          // staging slots per warp: 2 = the next block is copied while this one is unpacked
    int vpair;           // 64-token V blocks: an item is the pair of blocks of one token block (both channel halves)
    int kbound, vbound;  // largest legal block size in bytes
    int prow;            // bytes of one row of the score / probability tile
    int warp_smem;       // bytes of per-warp shared memory
    int off_xch, off_raw, off_perm, off_desc, off_stile, off_rst;   // byte offsets inside a warp's region
    int cta_off;         // byte offset of the CTA-shared block
    int out_off;         // byte offset, inside a warp's region, of its rows of the CTA's reduced output
    int tile_shift, cbk_shift, cbv_shift;   // log2 of tile, cbk, cbv
    int nkb_shift, nvi_shift;               // log2 of K blocks per tile and of V blocks (2 halves x token blocks) per tile
    FieldSpread klen, kmin, vlen, vmin;     // header field widths -> bytes
    AttnExchange x;      // head-sharded multi-GPU output exchange (n_ranks = 0: none)
    AttnAppend ap;       // the step's new token, written into residual row n_res - 1 by this launch (new_k = null: none)
    // two-launch form: `nsplit` clusters per (sequence, KV head), state handed over through caller scratch
    int nsplit;          // clusters per (sequence, KV head); 1 in the single-launch form
    int extra;           // two-launch form with cluster 1: the first `extra` pairs have nsplit + 1 CTAs, so that the CTAs of
                         // all pairs together fill the GPU's CTA slots exactly (grid = (total CTAs, 1, 1)); -1 = uniform
    int dump_bytes;      // bytes of a warp's score region (compressed + residual tiles), a multiple of 16
    unsigned* sc_count;  // [pairs] arrivals of the pair's clusters in the second launch (zero between launches)
    float* sc_ml;        // [pairs][cluster * nsplit][16] per-CTA max (8 rows) and sum (8 rows)
    uint8_t* sc_scores;  // [pairs][cluster * nsplit * kAW][dump_bytes]
    float* sc_part;      // [pairs][nsplit][8][kD] per-cluster unnormalised output rows
};

// CTA-shared block (cluster-visible)
struct CtaShared {
    float cl_m[8];       // this CTA's max per head
    float cl_l[8];       // this CTA's sum of exp(s - cl_m) per head
    float wm[kAW][8];    // per-warp scratch
    float gM[8], gInvL[8];
    unsigned lutm[8];    // (2^len - 1) * 0x00010001 per pack length 0..4 (see unpack8)
    unsigned last;       // two-launch form: this cluster is the pair's last one to deliver its rows
    unsigned pad_[3];
    unsigned long long mbar[kAW][2];
};
// The CTA's reduced accumulators out[head][channel] (read by rank 0 through distributed shared
// memory) live in the warps' regions, which are idle by then: head hd -> warp hd % kAW,
// float offset (hd / kAW) * kD (at most 8 / kAW rows of 512 bytes per warp: the 2 KB behind out_off hold them).
__device__ __forceinline__ float* cta_out_row(uint8_t* smem, int warp_smem, int out_off, int hd) {
    return reinterpret_cast<float*>(smem + (hd & (kAW - 1)) * warp_smem + out_off) + (hd / kAW) * kD;
}
static_assert(kAW == 1 || kAW == 2 || kAW == 4, "the reduced rows of a CTA must fit the warps' 2 KB regions");

// dequantise one register of two biased codes.  NORMAL: (code + zero) * scale with zadd = zero - bias (+ pack minimum);
// HP: code * scale + min, the product rounded before the addition as in the reference (_rn keeps the compiler
// from contracting the pair into one fused multiply-add), with cadd = pack minimum - bias.
template <typename T, bool HP>
__device__ __forceinline__ unsigned deq(unsigned biased, typename Tr<T>::T2 add, typename Tr<T>::T2 s, typename Tr<T>::T2 zmin) {
    using T2 = typename Tr<T>::T2;
    const T2 x = __hadd2(as_t2<T2>(biased), add);
    if (!HP) return as_u(__hmul2(x, s));
    return as_u(__hadd2(__hmul2_rn(x, s), zmin));
}

// =================================================================================================
// PASS: kFused = everything in one launch (one cluster per pair); kScores = first launch of the two-launch
// form: K phase, per-CTA max and sum and the score tiles go to the scratch; kValues = second launch: scores
// come back, global max and sum, V phase, per-cluster rows to the scratch, the pair's last cluster adds them up.
enum AttnPass : int { kFused = 0, kScores = 1, kValues = 2 };

template <typename T, int KMODE, bool HP, int PASS>
__global__ void __launch_bounds__(kAW * 32, PASS == 1 ? PKV_ATTN_CTAS_SCORES : PASS == 2 ? PKV_ATTN_CTAS_VALUES : kMaxCtasPerSm) attn_decode_kernel(const AttnDev P) {
    using T2 = typename Tr<T>::T2;
    constexpr unsigned MAGIC = Tr<T>::kMagic2;
    extern __shared__ __align__(16) uint8_t smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const AttnArgs& a = P.a;
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    // vrank: CTA index among all CTAs of the pair; n_vctas: how many the pair has; part_stride: rows of its scratch arrays
    int vrank = blockIdx.x, h = blockIdx.y, b = blockIdx.z, n_vctas = P.cluster * P.nsplit, part_stride = P.nsplit;
    if (PASS != kFused && P.extra >= 0) {
        // uneven form (cluster 1, one-dimensional grid): pairs 0 .. extra-1 have nsplit + 1 CTAs, the others nsplit
        const int c = blockIdx.x, big = P.extra * (P.nsplit + 1);
        int pr;
        if (c < big) { pr = c / (P.nsplit + 1); vrank = c - pr * (P.nsplit + 1); n_vctas = P.nsplit + 1; }
        else { const int c2 = c - big; pr = P.extra + c2 / P.nsplit; vrank = c2 % P.nsplit; n_vctas = P.nsplit; }
        b = pr / a.kv_heads; h = pr - b * a.kv_heads;
        part_stride = P.nsplit + 1;
    }
    const int rank = PASS == kFused ? vrank : vrank % P.cluster, split = PASS == kFused ? 0 : vrank / P.cluster;
    const int n_splits = n_vctas / P.cluster;          // clusters of this pair
    const int G = a.group;
    const int q_heads = a.kv_heads * G;
    const int n_warps = kAW * n_vctas;
    const int gw = vrank * kAW + wic;                  // warp index among all warps of the pair
    const int pair = b * a.kv_heads + h;
    const int ml_stride = P.cluster * part_stride;     // CTAs a pair's scratch rows are laid out for

    uint8_t* wbase = smem + wic * P.warp_smem;
    CtaShared* cs = reinterpret_cast<CtaShared*>(smem + P.cta_off);
    // 32-bit shared-window addresses for the hot loops
    const unsigned wbase_a = smem_addr(wbase);
    const unsigned xch_a = wbase_a + P.off_xch;        // K exchange: two tiles of 32 rows x 32 bytes
    const unsigned raw_a = wbase_a + P.off_raw;        // parameters as copied from global memory
    const unsigned perm_a = wbase_a + P.off_perm;      // per-token parameters in pair order: [tile] scale, [tile] zero
    const unsigned desc_a = wbase_a + P.off_desc;      // V: per channel-owner lane (pack offsets, lengths, minima)
    const unsigned stile_a = wbase_a + P.off_stile;    // [tpw][rows][prow] scores -> probabilities
    const unsigned rst_a = wbase_a + P.off_rst;        // [rtw][rows][16] residual scores -> probabilities
    unsigned lutm_a = smem_addr(cs->lutm);
    const unsigned bar_a = smem_addr(&cs->mbar[wic][0]);

    if (threadIdx.x < 5) {
        const unsigned L = threadIdx.x;
        cs->lutm[L] = ((1u << L) - 1u) * 0x00010001u;
    }
    if (lane == 0) {
        mbar_init(bar_a, 1);
        mbar_init(bar_a + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    asm volatile("" : "+r"(lutm_a) :: "memory");        // reads of the table stay behind the barrier

    const int my_tiles = gw < P.tiles_total ? (P.tiles_total - gw + n_warps - 1) / n_warps : 0;
    // residual tiles are dealt from the last warp backwards (the compressed tiles are dealt from
    // the first warp forwards, so the warps with one tile fewer take them)
    const int n_rt = (a.n_res + 15) >> 4, rslot = n_warps - 1 - gw;
    const int my_rt = rslot < n_rt ? (n_rt - rslot + n_warps - 1) / n_warps : 0;
    const int nkb = 1 << P.nkb_shift, nvi = 1 << P.nvi_shift;   // K blocks / V blocks per tile
    const int k_items = PASS == kValues ? 0 : my_tiles << P.nkb_shift, v_items = PASS == kScores ? 0 : my_tiles << P.nvi_shift;
    const int total_items = k_items + v_items;
    const int k_rounds = a.cbk >> 4;
    const int lbk = len_field_bits(a.bits_k), lbv = len_field_bits(a.bits_v);
    const uint8_t* kbase = a.k_stream + (int64_t)b * a.k_seq_stride;
    const uint8_t* vbase = a.v_stream + (int64_t)b * a.v_seq_stride;
    const T2 bias2 = Tr<T>::bias2();
    const T2 nbias2 = __hneg2(bias2);
    const T2 zmax2 = Tr<T>::zmax2();                   // largest zero-point for which (bias + code) + (zero - bias) is exact
    const bool col_live = 2 * c < P.rows;              // this lane's score columns (heads 2c, 2c+1) are kept
    const int ns_mask = P.nslots - 1;
    bool dead = false;                                 // a bounded wait gave up: this warp stops touching the stream
    bool bad_len = false, bad_zero = false;

    // ---- stream-block fetch ---------------------------------------------------------------------
    // Item n < k_items: K block (n % nkb) of local tile n / nkb.  Later items: V.  With 64-token V blocks an item is
    // the pair of blocks (both 64-channel halves of the head) of one token block, copied into the two halves of
    // the slot; with 128-token V blocks an item is one block.  An item's table entries are loaded one item ahead
    // of the copy that needs them.
    const uint2* kinfo_h = reinterpret_cast<const uint2*>(a.k_info) + (int64_t)b * a.k_info_seq_stride + h;
    const uint2* vinfo_h = reinterpret_cast<const uint2*>(a.v_info) + (int64_t)b * a.v_info_seq_stride + 2 * h;
    const T* kpar_s = reinterpret_cast<const T*>(a.k_scale) +
                      (KMODE == kKChannel ? (int64_t)(b * a.kv_heads + h) * a.param_blocks * kD : (int64_t)b * a.param_tokens);
    const T* kpar_z = reinterpret_cast<const T*>(a.k_zero) + (kpar_s - reinterpret_cast<const T*>(a.k_scale));
    const T* vpar_s = reinterpret_cast<const T*>(a.v_scale) + (int64_t)b * a.param_tokens;
    const T* vpar_z = reinterpret_cast<const T*>(a.v_zero) + (int64_t)b * a.param_tokens;
    const unsigned half_slot = (unsigned)P.slot >> 1;
    auto load_info = [&](int n) -> uint4 {
        if (n < k_items) {
            const int tl = n >> P.nkb_shift, i = n & (nkb - 1);
            const uint2 e = __ldg(kinfo_h + (((gw + tl * n_warps) << P.nkb_shift) + i) * a.kv_heads);
            return make_uint4(e.x, e.y, 0, 0);
        }
        const int m = n - k_items;
        const int tl = m >> P.nvi_shift, vi = m & (nvi - 1);
        if (P.vpair) {
            const uint2* p = vinfo_h + (((gw + tl * n_warps) << P.nvi_shift) + vi) * (2 * a.kv_heads);
            const uint2 e0 = __ldg(p), e1 = __ldg(p + 1);
            return make_uint4(e0.x, e0.y, e1.x, e1.y);
        }
        const uint2 e = __ldg(vinfo_h + (gw + tl * n_warps) * (2 * a.kv_heads) + vi);   // one 128-token block per tile: vi = half
        return make_uint4(e.x, e.y, 0, 0);
    };
    // (size << 4 | 16-byte phase) of a block that can be copied, 0 for a table entry that points outside the stream
    auto check_block = [&](unsigned off, unsigned size, const uint8_t* base, int64_t cap, int bound) -> unsigned {
        const bool bad = (int64_t)off + size > cap || (int)size > bound || size < 4 || ((off | size) & 1u);   // blocks start and end on even bytes
        return bad ? 0u : (size << 4) | (unsigned)(reinterpret_cast<uintptr_t>(base + off) & 15);
    };
    // Starts the copies of item n into its staging slot (same 16-byte phase as the source: block offsets are
    // arbitrary even bytes), together with the quantisation parameters the item needs: channel-mode K: the
    // block's 128 scales and 128 zero-points; token-mode K, first block of a tile: the tile's per-token scales
    // and zero-points; first V item of a tile: the same for V.  One lane issues, completion is counted in
    // bytes on the slot's mbarrier.
    auto issue = [&](int n, uint4 inf, unsigned& pk0, unsigned& pk1) {
        const T *p0 = nullptr, *p1 = nullptr;          // parameter sources
        unsigned pbytes = 0;
        const bool is_k = n < k_items;
        const uint8_t* base = is_k ? kbase : vbase;
        const int64_t cap = is_k ? a.k_capacity : a.v_capacity;
        const int bound = is_k ? P.kbound : P.vbound;
        if (is_k) {
            const int tl = n >> P.nkb_shift, i = n & (nkb - 1);
            if (KMODE == kKChannel) {
                const int off_e = (((gw + tl * n_warps) << P.nkb_shift) + i) * kD;
                p0 = kpar_s + off_e; p1 = kpar_z + off_e; pbytes = 2 * kD;
            } else if (i == 0) {
                const int t0 = (gw + tl * n_warps) << P.tile_shift;
                p0 = kpar_s + t0; p1 = kpar_z + t0; pbytes = 2 * P.tile;
            }
        } else {
            const int m = n - k_items;
            const int tl = m >> P.nvi_shift, vi = m & (nvi - 1);
            if (vi == 0 || (!P.vpair && vi == 0)) {
                const int t0 = (gw + tl * n_warps) << P.tile_shift;
                p0 = vpar_s + t0; p1 = vpar_z + t0; pbytes = 2 * P.tile;
            }
        }
        pk0 = check_block(inf.x, inf.y, base, cap, bound);
        pk1 = (!is_k && P.vpair) ? check_block(inf.z, inf.w, base, cap, bound) : 0u;
        if ((pk0 == 0 || (!is_k && P.vpair && pk1 == 0)) && lane == 0) atomicOr(a.flags, kFlagBadStream);
        if (lane == 0) {
            const unsigned slot = n & ns_mask;
            const unsigned dst = wbase_a + slot * P.slot, bar = bar_a + 8 * slot;
            const unsigned ph0 = pk0 & 15, tot0 = pk0 ? (ph0 + (pk0 >> 4) + 15) & ~15u : 0u;
            const unsigned ph1 = pk1 & 15, tot1 = pk1 ? (ph1 + (pk1 >> 4) + 15) & ~15u : 0u;
            mbar_expect_tx(bar, tot0 + tot1 + 2 * pbytes);
            if (tot0) bulk_g2s(dst, base + inf.x - ph0, tot0, bar);
            if (tot1) bulk_g2s(dst + half_slot, base + inf.z - ph1, tot1, bar);
            if (pbytes) {
                bulk_g2s(raw_a, p0, pbytes, bar);
                bulk_g2s(raw_a + (KMODE == kKChannel && is_k ? 2 * kD : 2 * P.tile), p1, pbytes, bar);
            }
        }
    };
    // with one slot the next item cannot be copied while this one is in use: it is pulled into L2 instead
    auto prefetch_l2 = [&](int n, uint4 inf2) {
        if (lane == 0) {
            const uint8_t* base = n < k_items ? kbase : vbase;
            const int64_t cap = n < k_items ? a.k_capacity : a.v_capacity;
            const unsigned bytes = inf2.y + inf2.w;       // a pair's blocks follow each other in the stream
            if ((int64_t)inf2.x + bytes <= cap && bytes <= 16384u && bytes >= 16u)
                bulk_prefetch_l2(reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(base + inf2.x) & ~(uintptr_t)15), bytes & ~15u);
        }
    };
    // all lanes wait for item n's copy; a wait that runs out marks the warp dead (it keeps reaching every barrier)
    auto wait_item = [&](int n) {
        if (dead) return;
        const unsigned bar = bar_a + 8 * (n & ns_mask), parity = (unsigned)(n >> (P.nslots - 1)) & 1u;
        if (!mbar_try_wait(bar, parity)) {
            unsigned spins = 0;
            while (!mbar_try_wait(bar, parity)) {
                if (++spins > kWaitSpins) { dead = true; break; }
            }
            dead = __any_sync(0xffffffffu, dead);
            if (dead && lane == 0) atomicOr(a.flags, kFlagTimeout);
        }
    };
    // natural-order per-token parameters (raw) -> pair order (perm); zero-points take the conversion bias
    auto permute_params = [&]() {
        const int quads = P.tile >> 2;                   // (group of eight, e) units per array
        if (lane < quads) {
            const int q8 = lane >> 1, e = lane & 1;
            const unsigned src = raw_a + 16 * q8 + 4 * e, dst = perm_a + 16 * q8 + 8 * (1 - e);
            unsigned w0, w1;
            pair_words(lds32(src), lds32(src + 8), w0, w1);
            sts64(dst, w0, w1);
            pair_words(lds32(src + 2 * P.tile), lds32(src + 2 * P.tile + 8), w0, w1);
            if (!HP) {
                // (bias + code) + (zero - bias) is exact while -bias <= zero and code + zero stays below 2 * bias
                const T2 z0 = as_t2<T2>(w0), z1 = as_t2<T2>(w1);
                if (!(__hbge2(z0, nbias2) && __hbge2(z1, nbias2) && __hble2(z0, zmax2) && __hble2(z1, zmax2))) bad_zero = true;
                w0 = as_u(__hsub2(z0, bias2)); w1 = as_u(__hsub2(z1, bias2));
            }
            sts64(dst + 2 * P.tile, w0, w1);
        }
        __syncwarp();
    };

    unsigned cur_pk0 = 0, cur_pk1 = 0, nxt_pk0 = 0, nxt_pk1 = 0;
    uint4 inf = make_uint4(0, 0, 0, 0);
    if (total_items > 0) issue(0, load_info(0), nxt_pk0, nxt_pk1);
    if (total_items > 1) inf = load_info(1);

    // q fragments for the compressed tiles.  The mma step (j, ap) contracts the 16 channels
    // 64 ap + 32 hf + 8 c' + 4 e + j  (k = 8 hf + 2 c' + e): plane j of the exchange tile, lanes 16 ap .. 16 ap + 15.
    // From the 8 consecutive elements x0..x7 of channels 32 m + 8 c.. (m = 2 ap + hf) the operand registers are
    // (x[j], x[j+4]).
    unsigned qf[4][2][2];
    {
        const uint4* qp = reinterpret_cast<const uint4*>(
            reinterpret_cast<const T*>(a.q) + ((int64_t)(b * q_heads + h * G + min(g, G - 1))) * kD + 8 * c);
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const uint4 v = g < G ? __ldg(qp + 4 * m) : make_uint4(0, 0, 0, 0);
            unsigned f0[2], f1[2];
            pair_shuffle(v, f0, f1);
            qf[0][m >> 1][m & 1] = f0[0]; qf[1][m >> 1][m & 1] = f0[1];
            qf[2][m >> 1][m & 1] = f1[0]; qf[3][m >> 1][m & 1] = f1[1];
        }
    }
    // exchange tile rows: lane l owns row l (32 bytes = 16 token slots) of the plane in flight; the two 16-byte
    // halves are swapped for rows 4..7 of every eight, which makes both the stores and the matrix loads conflict free
    const unsigned kst = xch_a + lane * 32, ksw = ((lane >> 2) & 1) << 4;
    unsigned kldm[2];
#pragma unroll
    for (int ap = 0; ap < 2; ap++) {
        const int row = 16 * ap + 8 * (lane >> 4) + (lane & 7), hf = (lane >> 3) & 1;
        kldm[ap] = xch_a + row * 32 + ((hf ^ ((row >> 2) & 1)) << 4);
    }
    // token (inside a round of 16) whose score this lane's fragment rows g and g+8 carry: slot g holds the low half
    // of the lower-row registers (6,2) (4,0) (14,10) (12,8), slot g + 8 the token after it
    const int tau = ((g >> 2) << 3) + ((g & 1) ? ((g & 2) ? 0 : 2) : ((g & 2) ? 4 : 6));

    T2 mpk0 = as_t2<T2>(Tr<T>::pack2(-INFINITY, -INFINITY)), mpk1 = mpk0;   // running max of this lane's scores, heads 2c and 2c+1

    // ============================================================================ phase 1: K tiles
    // one block: header, warp scan of the pack lengths, four packs per lane and round
    auto k_block = [&](auto bits_tag, unsigned blk, int i, unsigned st, const T2 (&ksd)[4], const T2 (&kzb)[4]) {
        constexpr int BK = decltype(bits_tag)::value, LBK = len_field_bits(BK);
        int pos = 2 * k_rounds;
        for (int r = 0; r < k_rounds; r++) {
            const unsigned hdr = blk + pos;
            unsigned lens4 = spread_const<LBK>(lane_word<4 * LBK>(hdr + 16 * BK, lane));   // byte j = length of pack j
            const unsigned mins4 = spread_const<BK>(lane_word<4 * BK>(hdr, lane));
            if ((lens4 + 0x03030303u) & 0x08080808u) { lens4 = 0; bad_len = true; }   // no encoder writes a length above 4
            const unsigned inc = warp_inclusive_sum(lens4);
            const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
            const unsigned exc2 = (inc - lens4) << 1;                 // byte j = byte offset of this lane's pack j in its group
            const unsigned packs = hdr + 16 * BK + 16 * LBK;
            unsigned pbase = packs;
            const int tk0 = (i << P.cbk_shift) + r * 16;              // first token of the round inside the tile
            uint4 sw[2], zw[2];                                       // token mode: parameter words of the round
            if (KMODE == kKToken) {
                sw[0] = lds128(perm_a + 2 * tk0); sw[1] = lds128(perm_a + 2 * tk0 + 16);
                zw[0] = lds128(perm_a + 2 * P.tile + 2 * tk0); zw[1] = lds128(perm_a + 2 * P.tile + 2 * tk0 + 16);
            }
            float accs[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};   // two chains hide the mma latency
#pragma unroll
            for (int j = 0; j < 4; j++) {
                unsigned lo, hi;
                ldp_u64_align2(pbase + byte_of(exc2, j), lo, hi);
                pbase += 2 * byte_of(tot, j);
                const unsigned len = byte_of(lens4, j);
                const unsigned m16 = ldp32(lutm_a + 4 * len);
                const unsigned s1 = 16u - 4u * len;
                unsigned ra[4], rb[4];
                unpack8<MAGIC>(__byte_perm(lo, hi, 0x3210u + 0x1111u * len), s1, len, m16, ra);   // tokens 0..7
                unpack8<MAGIC>(lo, s1, len, m16, rb);                                             // tokens 8..15
                // bias + pack minimum as an element pair, then the pack minimum alone
                const T2 mbf = __hadd2(as_t2<T2>(__byte_perm(mins4, Tr<T>::kMagicB, 0x4040 + 0x0101 * j)), nbias2);
                unsigned x[8];
                if (KMODE == kKChannel) {
                    const T2 add = HP ? __hadd2(mbf, nbias2) : __hadd2(kzb[j], mbf);
                    // in the order of the two stores below, so that each store's registers can be allocated in a row
                    x[1] = deq<T, HP>(ra[1], add, ksd[j], kzb[j]); x[3] = deq<T, HP>(ra[3], add, ksd[j], kzb[j]);
                    x[5] = deq<T, HP>(rb[1], add, ksd[j], kzb[j]); x[7] = deq<T, HP>(rb[3], add, ksd[j], kzb[j]);
                    x[0] = deq<T, HP>(ra[0], add, ksd[j], kzb[j]); x[2] = deq<T, HP>(ra[2], add, ksd[j], kzb[j]);
                    x[4] = deq<T, HP>(rb[0], add, ksd[j], kzb[j]); x[6] = deq<T, HP>(rb[2], add, ksd[j], kzb[j]);
                } else {
                    const unsigned s8[8] = {sw[0].x, sw[0].y, sw[0].z, sw[0].w, sw[1].x, sw[1].y, sw[1].z, sw[1].w};
                    const unsigned z8[8] = {zw[0].x, zw[0].y, zw[0].z, zw[0].w, zw[1].x, zw[1].y, zw[1].z, zw[1].w};
                    const T2 cadd = __hadd2(mbf, nbias2);
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        x[k] = deq<T, HP>(ra[k], HP ? cadd : __hadd2(as_t2<T2>(z8[k]), mbf), as_t2<T2>(s8[k]), as_t2<T2>(z8[k]));
                        x[4 + k] = deq<T, HP>(rb[k], HP ? cadd : __hadd2(as_t2<T2>(z8[4 + k]), mbf), as_t2<T2>(s8[4 + k]), as_t2<T2>(z8[4 + k]));
                    }
                }
                // slots 0..7: tokens 6 2 4 0 14 10 12 8; slots 8..15: the tokens after them
                const unsigned trow = kst + (j & 1) * 1024;
                sts128(trow + ksw, make_uint4(x[1], x[3], x[5], x[7]));
                sts128(trow + (ksw ^ 16), make_uint4(x[0], x[2], x[4], x[6]));
                __syncwarp();
#pragma unroll
                for (int ap = 0; ap < 2; ap++) {
                    unsigned af[4];
                    ldmatrix_x4_trans(kldm[ap] + (j & 1) * 1024, af);
                    Tr<T>::mma(accs[PKV_ONE_CHAIN ? 0 : ap], af, qf[j][ap][0], qf[j][ap][1]);
                }
            }
            // scores rounded like the reference: matmul output, then * scaling; fragment rows g and g + 8 are the
            // tokens tau and tau + 1, which share a store (lanes whose head columns are not kept compute too:
            // only the stores are predicated, no branch)
            {
                const unsigned row0 = st + (2 * c) * P.prow + 2 * (tk0 + tau);
                const unsigned p0 = Tr<T>::pack2(Tr<T>::round(accs[0][0] + accs[1][0]) * a.scaling, Tr<T>::round(accs[0][2] + accs[1][2]) * a.scaling);
                const unsigned p1 = Tr<T>::pack2(Tr<T>::round(accs[0][1] + accs[1][1]) * a.scaling, Tr<T>::round(accs[0][3] + accs[1][3]) * a.scaling);
                if (col_live) sts32(row0, p0);
                if (col_live) sts32(row0 + P.prow, p1);
                mpk0 = __hmax2(mpk0, as_t2<T2>(p0));
                mpk1 = __hmax2(mpk1, as_t2<T2>(p1));
            }
            pos += 16 * BK + 16 * LBK + (int)(pbase - packs);
        }
    };

    const T* kres = reinterpret_cast<const T*>(a.k_res) + (int64_t)b * a.res_seq_stride + (int64_t)h * a.res_head_stride;
    const T* vres = reinterpret_cast<const T*>(a.v_res) + (int64_t)b * a.res_seq_stride + (int64_t)h * a.res_head_stride;
    if constexpr (PASS != kValues) {
    for (int n = 0; n < k_items; n++) {
        cur_pk0 = nxt_pk0;
        wait_item(n);
        if (dead) cur_pk0 = 0;
        __syncwarp();
        // channel mode: scale and zero-point of this lane's four channels
        T2 ksd[4], kzb[4];
        if (KMODE == kKChannel) {
            const uint2 sv = lds64(raw_a + 8 * lane), zv = lds64(raw_a + 2 * kD + 8 * lane);
            ksd[0] = as_t2<T2>(__byte_perm(sv.x, 0, 0x1010)); ksd[1] = as_t2<T2>(__byte_perm(sv.x, 0, 0x3232));
            ksd[2] = as_t2<T2>(__byte_perm(sv.y, 0, 0x1010)); ksd[3] = as_t2<T2>(__byte_perm(sv.y, 0, 0x3232));
            if (!HP) {
                // (bias + code) + (zero - bias) is exact while -bias <= zero and code + zero stays below 2 * bias
                const T2 z01 = as_t2<T2>(zv.x), z23 = as_t2<T2>(zv.y);
                if (!(__hbge2(z01, nbias2) && __hbge2(z23, nbias2) && __hble2(z01, zmax2) && __hble2(z23, zmax2))) bad_zero = true;
                const unsigned y01 = as_u(__hsub2(z01, bias2)), y23 = as_u(__hsub2(z23, bias2));
                kzb[0] = as_t2<T2>(__byte_perm(y01, 0, 0x1010)); kzb[1] = as_t2<T2>(__byte_perm(y01, 0, 0x3232));
                kzb[2] = as_t2<T2>(__byte_perm(y23, 0, 0x1010)); kzb[3] = as_t2<T2>(__byte_perm(y23, 0, 0x3232));
            } else {
                kzb[0] = as_t2<T2>(__byte_perm(zv.x, 0, 0x1010)); kzb[1] = as_t2<T2>(__byte_perm(zv.x, 0, 0x3232));
                kzb[2] = as_t2<T2>(__byte_perm(zv.y, 0, 0x1010)); kzb[3] = as_t2<T2>(__byte_perm(zv.y, 0, 0x3232));
            }
            __syncwarp();                              // every lane has its parameters before the next copy lands
        }
        const int tl = n >> P.nkb_shift, i = n & (nkb - 1);
        if (KMODE == kKToken && i == 0 && !dead) permute_params();
        if (n + 1 < total_items && !dead) {
            if (P.nslots == 2) {
                issue(n + 1, inf, nxt_pk0, nxt_pk1);
                if (n + 2 < total_items) inf = load_info(n + 2);
            } else {
                prefetch_l2(n + 1, inf);
            }
        }
        unsigned blk = wbase_a + (n & ns_mask) * P.slot + (cur_pk0 & 15);
        asm volatile("" : "+r"(blk) :: "memory");          // the reads of the block stay behind the wait for its copy
        const unsigned st = stile_a + tl * P.rows * P.prow;
        if (cur_pk0 != 0 && !(PKV_ABL & 2)) {
            switch (a.bits_k) {
                case 4: k_block(std::integral_constant<int, 4>{}, blk, i, st, ksd, kzb); break;
                case 3: k_block(std::integral_constant<int, 3>{}, blk, i, st, ksd, kzb); break;
                default: k_block(std::integral_constant<int, 2>{}, blk, i, st, ksd, kzb); break;
            }
        }
        __syncwarp();
        if (P.nslots == 1 && n + 1 < total_items && !dead) {
            issue(n + 1, inf, nxt_pk0, nxt_pk1);
            if (n + 2 < total_items) inf = load_info(n + 2);
        }
    }
    float mloc0, mloc1;
    {
        const float2 m0 = Tr<T>::unpack2(as_u(mpk0)), m1 = Tr<T>::unpack2(as_u(mpk1));
        mloc0 = fmaxf(m0.x, m0.y); mloc1 = fmaxf(m1.x, m1.y);
    }

    // ---- residual tiles, phase 1: scores -------------------------------------------------------
    // A fragments come straight from the uncompressed rows: lane (g, c) reads channels
    // 32m + 8c .. +7 (m = 0..3) of tokens g and g+8 and pairs them in the order of pair_shuffle.
    // The decode step's new token: the warp that owns the residual tile of row n_res - 1 rotates K (the
    // arithmetic of rope_kernel: both products rounded to the element type, then their sum) and copies V into
    // that row first; its own loads of the tile below then see the row (plain loads and cp.async, no read-only path).
    if (P.ap.new_k != nullptr && my_rt > 0) {
        const int tn = a.n_res - 1, tile_n = tn >> 4;
        if (tile_n % n_warps == rslot) {
            if (lane < 16) {
                const T* x = reinterpret_cast<const T*>(P.ap.new_k) + (int64_t)b * P.ap.k_stride_b + (int64_t)h * P.ap.k_stride_h;
                const int d0 = 8 * lane;
                uint4 xv = *reinterpret_cast<const uint4*>(x + d0);
                if (P.ap.cos != nullptr) {
                    const uint4 rv = *reinterpret_cast<const uint4*>(x + (d0 < 64 ? d0 + 64 : d0 - 64));
                    const uint4 cv = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(P.ap.cos) + (int64_t)b * P.ap.cs_stride_b + d0);
                    const uint4 sv = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(P.ap.sin) + (int64_t)b * P.ap.cs_stride_b + d0);
                    const unsigned xs[4] = {xv.x, xv.y, xv.z, xv.w}, rs[4] = {rv.x, rv.y, rv.z, rv.w};
                    const unsigned cs4[4] = {cv.x, cv.y, cv.z, cv.w}, ss4[4] = {sv.x, sv.y, sv.z, sv.w};
                    unsigned o4[4];
                    const float sgn = d0 < 64 ? -1.f : 1.f;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 xf = Tr<T>::unpack2(xs[i]), rf = Tr<T>::unpack2(rs[i]), cf = Tr<T>::unpack2(cs4[i]), sf = Tr<T>::unpack2(ss4[i]);
                        const float a0 = Tr<T>::round(xf.x * cf.x), a1 = Tr<T>::round(xf.y * cf.y);
                        const float c0 = Tr<T>::round(sgn * rf.x * sf.x), c1 = Tr<T>::round(sgn * rf.y * sf.y);
                        o4[i] = Tr<T>::pack2(a0 + c0, a1 + c1);
                    }
                    xv = make_uint4(o4[0], o4[1], o4[2], o4[3]);
                }
                *reinterpret_cast<uint4*>(const_cast<T*>(kres) + (int64_t)tn * kD + d0) = xv;
            } else {
                const T* y = reinterpret_cast<const T*>(P.ap.new_v) + (int64_t)b * P.ap.v_stride_b + (int64_t)h * P.ap.v_stride_h;
                const int d0 = 8 * (lane - 16);
                *reinterpret_cast<uint4*>(const_cast<T*>(vres) + (int64_t)tn * kD + d0) = *reinterpret_cast<const uint4*>(y + d0);
            }
            __threadfence();
        }
        __syncwarp();
    }
    if (my_rt > 0) {
        unsigned qr[8][2];
        const uint4* qp = reinterpret_cast<const uint4*>(
            reinterpret_cast<const T*>(a.q) + ((int64_t)(b * q_heads + h * G + min(g, G - 1))) * kD + 8 * c);
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const uint4 v = g < G ? __ldg(qp + 4 * m) : make_uint4(0, 0, 0, 0);
            pair_shuffle(v, qr[2 * m], qr[2 * m + 1]);
        }
        for (int k = 0; k < my_rt; k++) {
            const int tok0 = (rslot + k * n_warps) << 4;
            const int ta = tok0 + g, tb = tok0 + g + 8;
            const uint4* pa = reinterpret_cast<const uint4*>(kres + (int64_t)min(ta, a.n_res - 1) * kD + 8 * c);
            const uint4* pb = reinterpret_cast<const uint4*>(kres + (int64_t)min(tb, a.n_res - 1) * kD + 8 * c);
            uint4 ra[4], rb[4];
#pragma unroll
            for (int m = 0; m < 4; m++) { ra[m] = pa[4 * m]; rb[m] = pb[4 * m]; }   // plain loads: a row may have been written by this launch
            float accs[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int m = 0; m < 4; m++) {
                unsigned a0[2], a1[2], b0[2], b1[2];
                pair_shuffle(ra[m], a0, a1);
                pair_shuffle(rb[m], b0, b1);
                const unsigned f0[4] = {a0[0], b0[0], a0[1], b0[1]};
                const unsigned f1[4] = {a1[0], b1[0], a1[1], b1[1]};
                Tr<T>::mma(accs[0], f0, qr[2 * m][0], qr[2 * m][1]);
                Tr<T>::mma(accs[1], f1, qr[2 * m + 1][0], qr[2 * m + 1][1]);
            }
            if (col_live) {
                const float ninf = -INFINITY;
                const float sa0 = ta < a.n_res ? Tr<T>::round(Tr<T>::round(accs[0][0] + accs[1][0]) * a.scaling) : ninf;
                const float sa1 = ta < a.n_res ? Tr<T>::round(Tr<T>::round(accs[0][1] + accs[1][1]) * a.scaling) : ninf;
                const float sb0 = tb < a.n_res ? Tr<T>::round(Tr<T>::round(accs[0][2] + accs[1][2]) * a.scaling) : ninf;
                const float sb1 = tb < a.n_res ? Tr<T>::round(Tr<T>::round(accs[0][3] + accs[1][3]) * a.scaling) : ninf;
                const unsigned row0 = rst_a + (k * P.rows + 2 * c) * 32 + 2 * g, row1 = row0 + 32;
                const T h00 = Tr<T>::from_float(sa0), h01 = Tr<T>::from_float(sa1), h10 = Tr<T>::from_float(sb0), h11 = Tr<T>::from_float(sb1);
                sts16(row0, *reinterpret_cast<const unsigned short*>(&h00)); sts16(row1, *reinterpret_cast<const unsigned short*>(&h01));
                sts16(row0 + 16, *reinterpret_cast<const unsigned short*>(&h10)); sts16(row1 + 16, *reinterpret_cast<const unsigned short*>(&h11));
                mloc0 = fmaxf(mloc0, fmaxf(sa0, sb0));
                mloc1 = fmaxf(mloc1, fmaxf(sa1, sb1));
            }
        }
    }

    // ---- warp max -> CTA max --------------------------------------------------------------------
#pragma unroll
    for (int d = 4; d < 32; d <<= 1) {
        mloc0 = fmaxf(mloc0, __shfl_xor_sync(0xffffffffu, mloc0, d));
        mloc1 = fmaxf(mloc1, __shfl_xor_sync(0xffffffffu, mloc1, d));
    }
    if (g == 0) {
        cs->wm[wic][2 * c] = mloc0;                     // columns >= rows carry -inf or the score of a zero q
        cs->wm[wic][2 * c + 1] = mloc1;
    }
    __syncthreads();
    if (threadIdx.x < 8) {
        float m = cs->wm[0][threadIdx.x];
#pragma unroll
        for (int w = 1; w < kAW; w++) m = fmaxf(m, cs->wm[w][threadIdx.x]);
        cs->cl_m[threadIdx.x] = m;
    }
    __syncthreads();
    // ---- sums relative to the CTA max: every lane takes one pair of tokens per row -------------
    {
        float lsum[8];
#pragma unroll
        for (int r = 0; r < 8; r++) lsum[r] = 0.f;
        const int chunks = P.tile >> 6;                  // 32 pairs per chunk
        for (int tl = 0; tl < my_tiles; tl++) {
            const unsigned st = stile_a + tl * P.rows * P.prow + 4 * lane;
#pragma unroll
            for (int r = 0; r < 8; r++) {
                if (r < P.rows) {
                    const float m = cs->cl_m[r];
                    for (int ch = 0; ch < chunks; ch++) {
                        const float2 x = Tr<T>::unpack2(lds32(st + r * P.prow + 128 * ch));
                        lsum[r] += fast_exp(x.x - m) + fast_exp(x.y - m);
                    }
                }
            }
        }
        if (lane < 8) {
            for (int k = 0; k < my_rt; k++) {
#pragma unroll
                for (int r = 0; r < 8; r++) {
                    if (r < P.rows) {
                        const float m = cs->cl_m[r];
                        const float2 x = Tr<T>::unpack2(lds32(rst_a + (k * P.rows + r) * 32 + 4 * lane));
                        // a masked token holds -inf; if the whole CTA is masked m is -inf too and the term must be 0
                        lsum[r] += (x.x == -INFINITY ? 0.f : fast_exp(x.x - m)) + (x.y == -INFINITY ? 0.f : fast_exp(x.y - m));
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 8; r++) {
            if (r < P.rows) {
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) lsum[r] += __shfl_xor_sync(0xffffffffu, lsum[r], d);
                if (lane == 0) cs->wm[wic][r] = lsum[r];   // wm's maxima were consumed before the barrier above
            }
        }
    }
    __syncthreads();
    if (threadIdx.x < 8) {
        float l = 0.f;
        if ((int)threadIdx.x < P.rows) {
#pragma unroll
            for (int w = 0; w < kAW; w++) l += cs->wm[w][threadIdx.x];
        }
        cs->cl_l[threadIdx.x] = l;
    }
    }   // PASS != kValues
    auto report_flags = [&]() {
        if (__any_sync(0xffffffffu, bad_len) && lane == 0) atomicOr(a.flags, kFlagBadStream);
        if (__any_sync(0xffffffffu, bad_zero) && lane == 0) atomicOr(a.flags, kFlagZeroRange);
    };
    if constexpr (PASS == kFused) {
        // ---- cluster exchange: global max and sum ---------------------------------------------------
        cluster.sync();
        if (threadIdx.x < 8) {
            float M = -INFINITY;
            for (int r = 0; r < P.cluster; r++) M = fmaxf(M, cluster.map_shared_rank(cs, r)->cl_m[threadIdx.x]);
            float L = 0.f;
            for (int r = 0; r < P.cluster; r++) {
                const CtaShared* o = cluster.map_shared_rank(cs, r);
                const float mr = o->cl_m[threadIdx.x];
                if (mr != -INFINITY) L += o->cl_l[threadIdx.x] * fast_exp(mr - M);
            }
            cs->gM[threadIdx.x] = M;
            cs->gInvL[threadIdx.x] = L > 0.f ? 1.f / L : 0.f;
        }
        __syncthreads();
    }
    if constexpr (PASS == kScores) {
        // ---- first launch ends here: this CTA's max and sum and every warp's score region go to the scratch ----
        // (the second launch may be set up from here on; it waits for this grid's completion before it reads anything)
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        __syncthreads();
        if (threadIdx.x < 16)
            P.sc_ml[((int64_t)pair * ml_stride + vrank) * 16 + threadIdx.x] = threadIdx.x < 8 ? cs->cl_m[threadIdx.x] : cs->cl_l[threadIdx.x - 8];
        {
            uint4* dst = reinterpret_cast<uint4*>(P.sc_scores + ((int64_t)pair * ml_stride * kAW + gw) * P.dump_bytes);
            const uint4* src = reinterpret_cast<const uint4*>(wbase + P.off_stile);
            for (int i = lane; i < (P.dump_bytes >> 4); i += 32) dst[i] = src[i];
        }
        report_flags();
        return;
    } else {
    if constexpr (PASS == kValues) {
        // ---- second launch starts here: the warp's score region comes back; global max and sum from all CTAs' ----
        // Launched with programmatic stream serialisation: everything above (barrier set-up, the copy of the first V
        // block) may overlap the first launch's tail; its results (scratch, the appended residual row) are read below.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        {
            const uint4* src = reinterpret_cast<const uint4*>(P.sc_scores + ((int64_t)pair * ml_stride * kAW + gw) * P.dump_bytes);
            uint4* dst = reinterpret_cast<uint4*>(wbase + P.off_stile);
            for (int i = lane; i < (P.dump_bytes >> 4); i += 32) dst[i] = __ldcg(src + i);
        }
        // thread t takes the CTAs t, t + 128, ...: maxima first, then the sums rescaled to the global maxima;
        // warp shuffles, then the four warps' values in a fixed order (every CTA of the pair gets the same bits)
        float m8[8], l8[8];
#pragma unroll
        for (int r = 0; r < 8; r++) { m8[r] = -INFINITY; l8[r] = 0.f; }
        const float4* ml = reinterpret_cast<const float4*>(P.sc_ml + (int64_t)pair * ml_stride * 16);
        for (int v = threadIdx.x; v < n_vctas; v += kAW * 32) {
            const float4 ma = __ldcg(ml + 4 * v), mb = __ldcg(ml + 4 * v + 1), la = __ldcg(ml + 4 * v + 2), lb = __ldcg(ml + 4 * v + 3);
            const float mv[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w}, lv[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
#pragma unroll
            for (int r = 0; r < 8; r++) {
                // one CTA per thread unless the pair has more than 128 of them: then rescale what is held already
                const float mn = fmaxf(m8[r], mv[r]);
                if (mn != -INFINITY) l8[r] = l8[r] * fast_exp(m8[r] - mn) + lv[r] * fast_exp(mv[r] - mn);
                m8[r] = mn;
            }
        }
        float M8[8];
#pragma unroll
        for (int r = 0; r < 8; r++) {
            float m = m8[r];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
            if (lane == 0) cs->wm[wic][r] = m;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 8; r++) {
            float m = cs->wm[0][r];
#pragma unroll
            for (int w = 1; w < kAW; w++) m = fmaxf(m, cs->wm[w][r]);
            M8[r] = m;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 8; r++) {
            float l = m8[r] != -INFINITY ? l8[r] * fast_exp(m8[r] - M8[r]) : 0.f;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) l += __shfl_xor_sync(0xffffffffu, l, d);
            if (lane == 0) cs->wm[wic][r] = l;
        }
        __syncthreads();
        if (threadIdx.x < 8) {
            float L = 0.f;
#pragma unroll
            for (int w = 0; w < kAW; w++) L += cs->wm[w][threadIdx.x];
            float M = -INFINITY;
#pragma unroll
            for (int r = 0; r < 8; r++) if (r == (int)threadIdx.x) M = M8[r];
            cs->gM[threadIdx.x] = M;
            cs->gInvL[threadIdx.x] = L > 0.f ? 1.f / L : 0.f;
        }
        __syncthreads();
    }

    // ============================================================================ phase 2: V tiles
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) o[i][j] = 0.f;

    // One V block (cbv tokens x 64 channels).  A segment is 64 tokens x 32 channels; lane l of the warp owns
    // channel l's four packs in the stream (lengths, minima, offsets), while the mma wants lane (g, c) to hold
    // channels g, g+8, g+16, g+24 for the 16 tokens of quarter c: the owners publish their pack descriptors
    // and every lane fetches the four packs its fragment rows need.
    // hh (which 64-channel half of the head) and w (which 32 channels of it) are compile-time, so that the accumulator
    // tiles a segment adds to are fixed registers and no branch selects them
    auto v_block = [&](auto bits_tag, auto hh_tag, unsigned blk, int tok_blk, unsigned st_a) {
        constexpr int BV = decltype(bits_tag)::value, LBV = len_field_bits(BV), HH = decltype(hh_tag)::value;
        const int rpw = a.cbv == 128 ? 2 : 1;           // segments of 64 tokens per 32 channels
        int pos = 4 * rpw;
        auto segment = [&](auto w_tag, int rr) {
            constexpr int W = decltype(w_tag)::value, SEL = 2 * HH + W;
            const int tok_seg = tok_blk + rr * 64;     // first token (in the tile) of the segment
            const unsigned hdr = blk + pos;
            unsigned lens4 = spread_const<LBV>(lane_word<4 * LBV>(hdr + 16 * BV, lane));   // byte q = length of pack q (tokens 16q..16q+15)
            const unsigned mins4 = spread_const<BV>(lane_word<4 * BV>(hdr, lane));
            if ((lens4 + 0x03030303u) & 0x08080808u) { lens4 = 0; bad_len = true; }
            const unsigned inc = warp_inclusive_sum(lens4);
            const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
            const unsigned packs = hdr + 16 * BV + 16 * LBV;
            sts32(desc_a + 4 * lane, (inc - lens4) << 1);
            sts32(desc_a + 128 + 4 * lane, lens4);
            sts32(desc_a + 256 + 4 * lane, mins4);
            // start of quarter c's packs: the quarters before it hold tot[0..c-1] halfwords
            const unsigned t01 = (tot & 0xFFu) + ((tot >> 8) & 0xFFu), t012 = t01 + ((tot >> 16) & 0xFFu);
            const unsigned before = c == 0 ? 0u : c == 1 ? (tot & 0xFFu) : c == 2 ? t01 : t012;
            const unsigned qbase = packs + 2 * before;
            __syncwarp();
            // per-token scale / zero pairs and probabilities for tokens tok_seg + 16c .. +15, in pair order
            const unsigned tok2 = 2 * (tok_seg + 16 * c);
            const uint4 s0 = lds128(perm_a + tok2), s1 = lds128(perm_a + tok2 + 16);
            const uint4 z0 = lds128(perm_a + 2 * P.tile + tok2), z1 = lds128(perm_a + 2 * P.tile + tok2 + 16);
            const unsigned vS[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            const unsigned vZ[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
            // head columns beyond the kept rows read a kept row: their output columns are never used
            const unsigned prow_a = st_a + min(g, P.rows - 1) * P.prow + tok2;
            const uint4 p0 = lds128(prow_a), p1 = lds128(prow_a + 16);
            const unsigned pw[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                unsigned x[2][8];                      // rows g (channel g + 16 mt) and g + 8 (channel g + 8 + 16 mt)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const unsigned da = desc_a + 4 * (g + 8 * (2 * mt + e)) + c;    // byte c of the owner's words
                    const unsigned len = lds8(da + 128);
                    unsigned lo, hi;
                    ldp_u64_align2(qbase + lds8(da), lo, hi);
                    const unsigned m16 = ldp32(lutm_a + 4 * len);
                    const unsigned sh1 = 16u - 4u * len;
                    unsigned ra[4], rb[4];
                    unpack8<MAGIC>(__byte_perm(lo, hi, 0x3210u + 0x1111u * len), sh1, len, m16, ra);
                    unpack8<MAGIC>(lo, sh1, len, m16, rb);
                    const T2 mbf = __hadd2(as_t2<T2>(__byte_perm(lds8(da + 256), Tr<T>::kMagicB, 0x4040)), nbias2);
                    const T2 cadd = __hadd2(mbf, nbias2);
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        x[e][k] = deq<T, HP>(ra[k], HP ? cadd : __hadd2(as_t2<T2>(vZ[k]), mbf), as_t2<T2>(vS[k]), as_t2<T2>(vZ[k]));
                        x[e][4 + k] = deq<T, HP>(rb[k], HP ? cadd : __hadd2(as_t2<T2>(vZ[4 + k]), mbf), as_t2<T2>(vS[4 + k]), as_t2<T2>(vZ[4 + k]));
                    }
                }
                // four steps of 16 token slots: step s takes the words 2s and 2s+1 of every quarter
#pragma unroll
                for (int s = 0; s < 4; s++) {
                    const unsigned af[4] = {x[0][2 * s], x[1][2 * s], x[0][2 * s + 1], x[1][2 * s + 1]};
                    Tr<T>::mma(o[2 * SEL + mt], af, pw[2 * s], pw[2 * s + 1]);
                }
            }
            __syncwarp();                              // descriptors are rewritten by the next segment
            pos += 16 * BV + 16 * LBV + 2 * (int)(t012 + (tot >> 24));
        };
        // (unrolling these two loops as well was measured slower: 122 against 117 us per layer)
#pragma unroll 1
        for (int rr = 0; rr < rpw; rr++) segment(std::integral_constant<int, 0>{}, rr);
#pragma unroll 1
        for (int rr = 0; rr < rpw; rr++) segment(std::integral_constant<int, 1>{}, rr);
    };

    for (int n = k_items; n < total_items; n++) {
        cur_pk0 = nxt_pk0; cur_pk1 = nxt_pk1;
        wait_item(n);
        if (dead) { cur_pk0 = 0; cur_pk1 = 0; }
        __syncwarp();
        const int m = n - k_items;
        const int tl = m >> P.nvi_shift, vi = m & (nvi - 1);
        const unsigned st_a = stile_a + tl * P.rows * P.prow;

        if (vi == 0 && !dead) {
            // the tile's V scales and zero-points, pair order
            permute_params();
            // scores -> probabilities rounded to the element type, in place, pair order: unit u = (row, group of
            // eight tokens, e); loads of up to four units per lane, a warp barrier, then the stores
            const int pr_shift = P.tile_shift - 2, units = P.rows << pr_shift;
            for (int u0 = 0; u0 < units; u0 += 128) {
                unsigned w0[4], w1[4];
#pragma unroll
                for (int it = 0; it < 4; it++) {
                    const int u = u0 + 32 * it + lane;
                    if (u < units) {
                        const int r = u >> pr_shift, rem = u & ((1 << pr_shift) - 1), q8 = rem >> 1, e = rem & 1;
                        const unsigned ad = st_a + r * P.prow + 16 * q8 + 4 * e;
                        const float M = cs->gM[r], I = cs->gInvL[r];
                        const float2 xa = Tr<T>::unpack2(lds32(ad)), xb = Tr<T>::unpack2(lds32(ad + 8));
                        const unsigned pa = Tr<T>::pack2(fast_exp(xa.x - M) * I, fast_exp(xa.y - M) * I);
                        const unsigned pb = Tr<T>::pack2(fast_exp(xb.x - M) * I, fast_exp(xb.y - M) * I);
                        pair_words(pa, pb, w0[it], w1[it]);
                    }
                }
                __syncwarp();
#pragma unroll
                for (int it = 0; it < 4; it++) {
                    const int u = u0 + 32 * it + lane;
                    if (u < units) {
                        const int r = u >> pr_shift, rem = u & ((1 << pr_shift) - 1), q8 = rem >> 1, e = rem & 1;
                        sts64(st_a + r * P.prow + 16 * q8 + 8 * (1 - e), w0[it], w1[it]);
                    }
                }
                __syncwarp();
            }
        }
        if (n + 1 < total_items && !dead) {
            if (P.nslots == 2) {
                issue(n + 1, inf, nxt_pk0, nxt_pk1);
                if (n + 2 < total_items) inf = load_info(n + 2);
            } else {
                prefetch_l2(n + 1, inf);
            }
        }
        unsigned sbase = wbase_a + (n & ns_mask) * P.slot;
        asm volatile("" : "+r"(sbase) :: "memory");        // the reads of the blocks stay behind the wait for their copy
        if (!(PKV_ABL & 1)) {
#pragma unroll 1
            for (int sub = 0; sub < (P.vpair ? 2 : 1); sub++) {
                const unsigned pk = sub ? cur_pk1 : cur_pk0;
                if (pk == 0) continue;
                const unsigned blk = sbase + sub * half_slot + (pk & 15);
                const int hh = P.vpair ? sub : vi;                       // which 64-channel half of the head
                const int tok_blk = P.vpair ? (vi << 6) : 0;             // token offset of the block in the tile
                auto by_half = [&](auto bits_tag) {
                    if (hh) v_block(bits_tag, std::integral_constant<int, 1>{}, blk, tok_blk, st_a);
                    else v_block(bits_tag, std::integral_constant<int, 0>{}, blk, tok_blk, st_a);
                };
                switch (a.bits_v) {
                    case 4: by_half(std::integral_constant<int, 4>{}); break;
                    case 3: by_half(std::integral_constant<int, 3>{}); break;
                    default: by_half(std::integral_constant<int, 2>{}); break;
                }
            }
        }
        __syncwarp();
        if (P.nslots == 1 && n + 1 < total_items && !dead) {
            issue(n + 1, inf, nxt_pk0, nxt_pk1);
            if (n + 2 < total_items) inf = load_info(n + 2);
        }
    }
    __syncwarp();
    report_flags();

    // ---- residual tiles, phase 2: probabilities x V ---------------------------------------------
    // The tile's 16 V rows are staged (padded to 272 bytes so that ldmatrix is conflict free) in the
    // idle staging slots; ldmatrix.trans turns them into channels x tokens A fragments.
    for (int k = 0; k < my_rt; k++) {
        const int tok0 = (rslot + k * n_warps) << 4;
        __syncwarp();
        for (int j = lane; j < 256; j += 32) {           // 16 rows x 16 chunks of 16 bytes
            const int row = j >> 4, chunk = j & 15;
            const bool live = tok0 + row < a.n_res;
            cp_async16_zfill(wbase_a + row * 272 + chunk * 16, vres + (int64_t)(live ? tok0 + row : 0) * kD + 8 * chunk, live);
        }
        cp_async_commit();
        if (lane < 8) {
#pragma unroll
            for (int r = 0; r < 8; r++) {
                if (r < P.rows) {
                    const float M = cs->gM[r], I = cs->gInvL[r];
                    const unsigned ad = rst_a + (k * P.rows + r) * 32 + 4 * lane;
                    const float2 x = Tr<T>::unpack2(lds32(ad));
                    sts32(ad, Tr<T>::pack2(x.x == -INFINITY ? 0.f : fast_exp(x.x - M) * I, x.y == -INFINITY ? 0.f : fast_exp(x.y - M) * I));
                }
            }
        }
        cp_async_wait<0>();
        __syncwarp();
        unsigned b0 = 0, b1 = 0;
        if (g < P.rows) {
            b0 = lds32(rst_a + (k * P.rows + g) * 32 + 4 * c);
            b1 = lds32(rst_a + (k * P.rows + g) * 32 + 4 * c + 16);
        }
        // matrix m of the x4 load: tokens 8*(m>>1).., channels 16*mt + 8*(m&1)..
        const unsigned lm = wbase_a + (((lane >> 4) << 3) + (lane & 7)) * 272 + (((lane >> 3) & 1) << 4);
#pragma unroll
        for (int mt = 0; mt < 8; mt++) {
            unsigned af[4];
            ldmatrix_x4_trans(lm + 32 * mt, af);
            Tr<T>::mma(o[mt], af, b0, b1);
        }
    }
    __syncwarp();
    // a launch that follows under programmatic stream serialisation (the exchange's wait) may be set up from here on
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // ---- warp accumulators -> this warp's shared region: red[head][channel] --------------------
    float* red = reinterpret_cast<float*>(wbase);
#pragma unroll
    for (int mt = 0; mt < 8; mt++) {
        red[(2 * c) * kD + 16 * mt + g] = o[mt][0];
        red[(2 * c + 1) * kD + 16 * mt + g] = o[mt][1];
        red[(2 * c) * kD + 16 * mt + g + 8] = o[mt][2];
        red[(2 * c + 1) * kD + 16 * mt + g + 8] = o[mt][3];
    }
    __syncwarp();
    __syncthreads();
    // ---- CTA reduce, then cluster reduce on rank 0 ---------------------------------------------
    constexpr int kThreads = kAW * 32;
    for (int d = threadIdx.x; d < kD; d += kThreads) {
        for (int hd = 0; hd < G; hd++) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kAW; w++) v += reinterpret_cast<const float*>(smem + w * P.warp_smem)[hd * kD + d];
            cta_out_row(smem, P.warp_smem, P.out_off, hd)[d] = v;
        }
    }
    cluster.sync();
    if (rank == 0) {
        bool deliver = true;
        if constexpr (PASS == kValues) {
            // this cluster's rows go to the scratch; the cluster that finds all the others' there adds them up
            float* part = P.sc_part + ((int64_t)pair * part_stride + split) * 8 * kD;
            for (int d = threadIdx.x; d < kD; d += kThreads) {
                for (int hd = 0; hd < G; hd++) {
                    float v = 0.f;
                    for (int r = 0; r < P.cluster; r++) v += cluster.map_shared_rank(cta_out_row(smem, P.warp_smem, P.out_off, hd), r)[d];
                    __stcg(part + hd * kD + d, v);
                }
            }
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) cs->last = atomicAdd(P.sc_count + pair, 1u) == (unsigned)(n_splits - 1) ? 1u : 0u;
            __syncthreads();
            deliver = cs->last != 0;
            if (deliver) __threadfence();
        }
        if (deliver) {
            for (int d = threadIdx.x; d < kD; d += kThreads) {
                for (int hd = 0; hd < G; hd++) {
                    float v = 0.f;
                    if constexpr (PASS == kValues) {
                        for (int sp = 0; sp < n_splits; sp++) v += __ldcg(P.sc_part + (((int64_t)pair * part_stride + sp) * 8 + hd) * kD + d);
                    } else {
                        for (int r = 0; r < P.cluster; r++) v += cluster.map_shared_rank(cta_out_row(smem, P.warp_smem, P.out_off, hd), r)[d];
                    }
                    const T r = Tr<T>::from_float(v);
                    const int64_t idx = ((int64_t)(b * q_heads + h * G + hd)) * kD + d;
                    reinterpret_cast<T*>(a.out)[idx] = r;
                    // head-sharded decode: the same row goes into this rank's slice of every rank's gathered buffer
                    for (int p = 0; p < P.x.n_ranks; p++)
                        reinterpret_cast<T*>(P.x.gathered[p])[(int64_t)P.x.rank * a.batch * q_heads * kD + idx] = r;
                }
            }
            if (PASS == kValues && threadIdx.x == 0) P.sc_count[pair] = 0u;   // ready for the next launch on this scratch
            if (P.x.n_ranks > 0) {
                __threadfence_system();                // the rows are visible to the other GPUs before the arrival is
                __syncthreads();
                if ((int)threadIdx.x < P.x.n_ranks) atomicAdd_system(P.x.arrivals[threadIdx.x] + P.x.rank, 1u);
            }
        }
    }
    cluster.sync();   // keep every CTA's shared memory alive until rank 0 has read it
    }   // PASS != kScores
}

// =================================================================================================
static int k_bound(int cb, int bits) { int r = cb / 16; return 2 * r + r * (16 * bits + 16 * len_field_bits(bits) + 256 * bits); }
static int v_bound(int cb, int bits) { int n = cb == 128 ? 4 : 2; return 2 * n + n * (16 * bits + 16 * len_field_bits(bits) + 256 * bits); }

// tuning overrides read once from the environment (0 = choose automatically)
static int env_int(const char* name) {
    const char* v = std::getenv(name);
    return v ? std::atoi(v) : 0;
}

template <typename T, int KM, bool HPV, int PASS>
static int launch_one(const AttnDev& P, dim3 grid, int smem, cudaStream_t st) {
    auto kern = attn_decode_kernel<T, KM, HPV, PASS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kCudaError;
    if (P.cluster > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) return kCudaError;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kAW * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = P.cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (PASS == kValues) {
        // the second launch may start while the first one drains; it waits for it on the device (griddepcontrol.wait)
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    if (P.cluster > 8) {
        // a non-portable cluster size with this much shared memory may not be schedulable at all: say so
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return kCudaError; }
        if (clusters < 1) return kUnsupported;
    }
    return cudaLaunchKernelEx(&cfg, kern, P) == cudaSuccess ? kOk : kCudaError;
}

template <typename T, int PASS>
static int launch_pass(const AttnDev& P, dim3 grid, int smem, cudaStream_t st) {
    const AttnArgs& a = P.a;
    if (a.k_mode == kKChannel)
        return a.high_precision_zero ? launch_one<T, kKChannel, true, PASS>(P, grid, smem, st) : launch_one<T, kKChannel, false, PASS>(P, grid, smem, st);
    return a.high_precision_zero ? launch_one<T, kKToken, true, PASS>(P, grid, smem, st) : launch_one<T, kKToken, false, PASS>(P, grid, smem, st);
}

template <typename T>
static int launch_typed(const AttnDev& P, dim3 grid, int smem, cudaStream_t st) {
    if (P.nsplit == 1 && P.sc_count == nullptr) return launch_pass<T, kFused>(P, grid, smem, st);
#ifdef PKV_DEBUG_PASS   // measurement builds: one of the two launches alone (the results are then meaningless)
    static const int only = env_int("PKV_ATTN_ONLY_PASS");
    if (only == 1) return launch_pass<T, kScores>(P, grid, smem, st);
    if (only == 2) return launch_pass<T, kValues>(P, grid, smem, st);
#endif
    const int rc = launch_pass<T, kScores>(P, grid, smem, st);
    return rc != kOk ? rc : launch_pass<T, kValues>(P, grid, smem, st);
}


// shared memory of one CTA for a cluster of `cl` CTAs with `nslots` staging slots per warp; fills the layout fields
static int plan_smem(AttnDev& P, int cl, int nsplit, int nslots, int slot) {
    const AttnArgs& a = P.a;
    const int n_warps = kAW * cl * nsplit;
    P.cluster = cl;
    P.nsplit = nsplit;
    P.nslots = nslots;
    P.slot = slot;
    P.tpw = (P.tiles_total + n_warps - 1) / n_warps;
    P.rtw = ((a.n_res + 15) / 16 + n_warps - 1) / n_warps;
    int off = nslots * slot;
    if (off < 16 * 272) off = 16 * 272;                       // the residual V tile borrows the staging slots
    if (off < 8 * kD * 4) off = 8 * kD * 4;                   // and so do the parked accumulators
    P.out_off = off;                                          // the CTA's reduced rows sit behind them
    P.off_xch = off; off += 2048;                             // (>= 2 * kD * 4 bytes: two heads' rows per warp)
    // The parameter staging, the pair-order parameters and the V descriptors are idle while the K exchange tile
    // is in use when K has per-channel parameters and the next item is only copied after the current one is
    // done (one slot): the parameters of a block are in registers before its first round.  They share the tile then.
    const int raw_bytes = 4 * P.tile > 4 * kD ? 4 * P.tile : 4 * kD;
    if (a.k_mode == kKChannel && nslots == 1 && raw_bytes + 4 * P.tile + 384 <= 2048) {
        P.off_raw = P.off_xch; P.off_perm = P.off_raw + raw_bytes; P.off_desc = P.off_perm + 4 * P.tile;
    } else {
        P.off_raw = off; off += raw_bytes;
        P.off_perm = off; off += 4 * P.tile;
        P.off_desc = off; off += 384;
    }
    P.off_stile = off; off += P.tpw * P.rows * P.prow;
    P.off_rst = off; off += P.rtw * P.rows * 32;
    P.warp_smem = (off + 15) & ~15;
    P.dump_bytes = P.warp_smem - P.off_stile;
    P.cta_off = kAW * P.warp_smem;
    return P.cta_off + (int)sizeof(CtaShared);
}

// partition of the caller's scratch for the two-launch form
struct ScratchLayout { int64_t count, ml, part, scores, total; };
static ScratchLayout scratch_layout(int64_t pairs, int cl, int nsplit, int dump_bytes) {   // nsplit: the largest of any pair
    ScratchLayout L;
    int64_t off = 0;
    L.count = off; off += (pairs * 4 + 255) & ~(int64_t)255;
    L.ml = off; off += pairs * cl * nsplit * 64;
    L.part = off; off += pairs * nsplit * 8 * kD * 4;
    off = (off + 255) & ~(int64_t)255;
    L.scores = off; off += pairs * cl * nsplit * kAW * (int64_t)dump_bytes;
    L.total = off;
    return L;
}

// One warp polls this rank's arrival counters; see pkv_exchange_wait.  consume: once every counter has reached
// `expected`, that many arrivals are taken off it again, so that the same launch (same `expected`) serves every step:
// what a CUDA graph over the layer loop needs.
__global__ void exchange_wait_kernel(uint32_t* arrivals, int n_ranks, unsigned expected, unsigned max_polls, unsigned* flags, int consume) {
    const int lane = threadIdx.x;
    bool ok = lane >= n_ranks;
    for (unsigned it = 0; it <= max_polls; it++) {
        if (!ok) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(arrivals + lane) : "memory");
            ok = (int)(v - expected) >= 0;
        }
        if (__all_sync(0xffffffffu, ok)) break;
        __nanosleep(250);
    }
    const bool all = __all_sync(0xffffffffu, ok);
    if (!all && lane == 0) atomicOr(flags, kFlagTimeout);
    if (all && consume && lane < n_ranks) atomicSub(arrivals + lane, expected);   // resolved where the peers' additions are: this GPU's L2
    __threadfence_system();
}

int launch_exchange_wait(uint32_t* arrivals, int n_ranks, unsigned expected, unsigned max_polls, unsigned* flags, bool consume, cudaStream_t st) {
    if (!arrivals || !flags || n_ranks < 1 || n_ranks > 8) return kBadArgument;
    // The wait needs nothing from the launch before it but this rank's own arrivals, which are counted like the
    // others': it may start while that launch drains (programmatic stream serialisation, no device-side wait) and
    // ends when the last rank has arrived.  Launches after it are ordered behind both.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, 1);
    cfg.blockDim = dim3(32, 1, 1);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, exchange_wait_kernel, arrivals, n_ranks, expected, max_polls, flags, consume ? 1 : 0) != cudaSuccess) {
        cudaGetLastError();
        return kCudaError;
    }
    return kOk;
}

// plan_io: in: cluster / nsplit / launches to force (0 = choose); out: what was chosen.  dry_run: plan only.
int launch_attention(const AttnArgs& a, const AttnExchange* xch, const AttnAppend* ap, AttnPlan* plan_io, void* scratch, int64_t scratch_bytes,
                     bool dry_run, cudaStream_t st) {
    if (a.batch <= 0 || a.kv_heads <= 0 || a.group < 1 || a.group > 8) return a.group > 8 ? kUnsupported : kBadArgument;
    if (a.n_comp < 0 || a.n_res < 0 || a.n_comp + a.n_res == 0) return kBadArgument;
    if (!a.q || !a.out || !a.flags) return kBadArgument;
    if (a.n_comp > 0) {
        if ((a.cbk != 64 && a.cbk != 128) || (a.cbv != 64 && a.cbv != 128)) return kUnsupported;
        if (a.bits_k < 2 || a.bits_k > 4 || a.bits_v < 2 || a.bits_v > 4) return kUnsupported;
        if (a.k_mode != kKChannel && a.k_mode != kKToken) return kUnsupported;
        const int tile = (a.cbk == 128 || a.cbv == 128) ? 128 : 64;
        if (a.n_comp % tile) return kBadArgument;
        if (a.param_tokens < a.n_comp || (a.k_mode == kKChannel && a.param_blocks < a.n_comp / a.cbk)) return kBadArgument;
        if (!a.k_stream || !a.k_info || !a.k_scale || !a.k_zero || !a.v_stream || !a.v_info || !a.v_scale || !a.v_zero) return kBadArgument;
        if ((reinterpret_cast<uintptr_t>(a.k_stream) & 15) || (a.k_seq_stride & 15) || (reinterpret_cast<uintptr_t>(a.v_stream) & 15) ||
            (a.v_seq_stride & 15) || (a.k_capacity & 15) || (a.v_capacity & 15))
            return kBadArgument;
        if ((reinterpret_cast<uintptr_t>(a.k_scale) & 15) || (reinterpret_cast<uintptr_t>(a.k_zero) & 15)) return kBadArgument;
        if ((reinterpret_cast<uintptr_t>(a.v_scale) & 15) || (reinterpret_cast<uintptr_t>(a.v_zero) & 15) || (a.param_tokens & 7)) return kBadArgument;
        if ((reinterpret_cast<uintptr_t>(a.k_info) & 7) || (reinterpret_cast<uintptr_t>(a.v_info) & 7)) return kBadArgument;
    }
    if (a.n_res > 0) {
        if (!a.k_res || !a.v_res) return kBadArgument;
        if ((reinterpret_cast<uintptr_t>(a.k_res) & 15) || (reinterpret_cast<uintptr_t>(a.v_res) & 15) || (a.res_seq_stride & 7) || (a.res_head_stride & 7))
            return kBadArgument;
    }
    if (reinterpret_cast<uintptr_t>(a.q) & 15) return kBadArgument;

    AttnDev P{};
    P.extra = -1;
    P.a = a;
    if (ap) {
        if (!ap->new_k || !ap->new_v || a.n_res < 1 || a.n_res > ap->res_capacity || ((ap->cos == nullptr) != (ap->sin == nullptr))) return kBadArgument;
        if ((reinterpret_cast<uintptr_t>(ap->new_k) & 15) || (reinterpret_cast<uintptr_t>(ap->new_v) & 15) || (ap->k_stride_b & 7) || (ap->k_stride_h & 7) ||
            (ap->v_stride_b & 7) || (ap->v_stride_h & 7) || (reinterpret_cast<uintptr_t>(ap->cos) & 15) || (reinterpret_cast<uintptr_t>(ap->sin) & 15) ||
            (ap->cs_stride_b & 7))
            return kBadArgument;
        P.ap = *ap;
    }
    if (xch) {
        if (xch->n_ranks < 1 || xch->n_ranks > 8 || xch->rank < 0 || xch->rank >= xch->n_ranks) return kBadArgument;
        for (int p = 0; p < xch->n_ranks; p++)
            if (!xch->gathered[p] || !xch->arrivals[p]) return kBadArgument;
        P.x = *xch;
    }
    P.tile = (a.n_comp > 0 && (a.cbk == 128 || a.cbv == 128)) ? 128 : 64;
    P.tiles_total = a.n_comp / P.tile;
    auto lg2 = [](int v) { int s = 0; while ((1 << s) < v) s++; return s; };
    P.tile_shift = lg2(P.tile);
    P.cbk_shift = a.n_comp > 0 ? lg2(a.cbk) : 6;
    P.cbv_shift = a.n_comp > 0 ? lg2(a.cbv) : 6;
    P.nkb_shift = P.tile_shift - P.cbk_shift;
    P.vpair = a.n_comp > 0 && a.cbv == 64;
    P.nvi_shift = P.vpair ? P.tile_shift - 6 : 1;   // V items per tile: token blocks of 64 (as pairs) or the two halves of a 128-token block
    if (a.n_comp > 0) {
        P.klen = make_field_spread(len_field_bits(a.bits_k)); P.kmin = make_field_spread(a.bits_k);
        P.vlen = make_field_spread(len_field_bits(a.bits_v)); P.vmin = make_field_spread(a.bits_v);
    }
    P.rows = (a.group + 1) & ~1;
    P.prow = 2 * P.tile + 16;
    int slot = 0;
    if (a.n_comp > 0) {
        const int kb = k_bound(a.cbk, a.bits_k), vb = v_bound(a.cbv, a.bits_v);
        P.kbound = kb; P.vbound = vb;
        const int ks = (kb + 48 + 15) & ~15;                   // 15 bytes of phase, 16 of round-up, window reads past the end
        const int vs = P.vpair ? 2 * ((vb + 48 + 15) & ~15) : (vb + 48 + 15) & ~15;
        slot = ((ks > vs ? ks : vs) + 31) & ~31;                // the halves of a slot are 16-byte aligned
    }
    // Cluster size, clusters per pair and staging depth: the (sequence, KV head) pairs times their CTAs should
    // fill the 148 SMs' CTA slots in whole waves, every warp should have work, and a warp's scores must fit in
    // shared memory.  Cost model: waves x (work units per warp + a fixed part) x (resident warps beyond about 9
    // per SM share the issue slots).  Several clusters per pair need the scratch and two launches.
    static const int env_cl = env_int("PKV_ATTN_CLUSTER"), env_slots = env_int("PKV_ATTN_SLOTS");
    const int want_cl = plan_io && plan_io->cluster > 0 ? plan_io->cluster : env_cl;
    const int want_split = plan_io && plan_io->nsplit > 0 ? plan_io->nsplit : 0;
    const int want_launches = plan_io ? plan_io->launches : 0;
    const int want_extra = plan_io ? plan_io->extra : 0;
    if (want_cl < 0 || want_cl > 16 || want_launches < 0 || want_launches > 2 || want_extra < 0) return kBadArgument;
    if (scratch && ((reinterpret_cast<uintptr_t>(scratch) & 255) || scratch_bytes < 0)) return kBadArgument;
    const long pairs = (long)a.batch * a.kv_heads;
    const int unit_tile = (P.tile / 64) * 4;                   // a residual tile is about a quarter of 64 compressed tokens
    const int n_rt = (a.n_res + 15) / 16;
    const double pair_units = (double)P.tiles_total * unit_tile + n_rt;
    // Cost of a plan, in units of 16 tokens of one warp.  An SM's throughput stops growing at about 13 resident warps
    // (the kernel is bound by instruction issue), so the time of a launch follows the work of its busiest SM:
    // (warps on it) x (average units per warp + a fixed part) / min(warps, 13), and never less than the longest warp.
    // Fixed part: exchange and reductions; in two launches also the hand-over, a second start and one more row to add
    // per cluster of the pair.  Clusters are placed inside one GPC: about 7 % of the slots stay unusable for them
    // (136 clusters of 4 fit at once, 144 do not), and clusters above the portable size schedule badly once they
    // fill more than half the GPU.
    auto plan_cost = [&](long ctas, int cl, int per_sm, double avg_upw, int upw_max, double fixed, int ns) {
        long slots = (long)kSmCount * per_sm;
        if (cl > 1) slots = (long)((double)slots * 0.93 / cl) * cl;
        if (slots < cl) slots = cl;
        const long waves = (ctas + slots - 1) / slots;
        const long on_gpu = ctas < slots ? ctas : slots;
        const int sm_warps = (int)((on_gpu + kSmCount - 1) / kSmCount) * kAW;
        // (a launch ends with its longest warps running alone, below the saturated rate: three quarters of the
        // difference between the longest and the average warp count as if every warp had them)
        const double eff_upw = avg_upw + 0.75 * (upw_max - avg_upw);
        const double thr = sm_warps * (eff_upw + fixed) / (sm_warps < 13 ? sm_warps : 13);
        const double lat = upw_max + fixed;
        double cost = (double)waves * (thr > lat ? thr : lat);
        if (ns == 1) cost *= 1.02;                              // the copy of the next block is not overlapped (it comes from L2)
        if (cl > 8) cost *= 2 * ctas > slots ? 1.4 : 1.1;
        return cost;
    };
    static const int kSplits[] = {1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64};
    int best_cl = 0, best_ns = 1, best_split = 1, best_launches = 1, best_extra = -1;
    double best_cost = 1e300;
    for (int cl = 1; cl <= 16 && want_extra == 0; cl++) {
        if (want_cl && cl != want_cl) continue;
        for (int split : kSplits) {
            if (want_split && split != want_split) continue;
            if (cl * split > 128) continue;
            for (int launches = 1; launches <= 2; launches++) {
                if (want_launches && launches != want_launches) continue;
                if (launches == 1 && split > 1) continue;
                if (launches == 2 && split == 1 && want_launches != 2) continue;   // one cluster in two launches: only on request
                for (int ns = 2; ns >= 1; ns--) {
                    if (env_slots && ns != env_slots) continue;
                    AttnDev Q = P;
                    const int smem = plan_smem(Q, cl, split, ns, slot);
                    if (smem > 227 * 1024) continue;
                    if (launches == 2 && (!scratch || scratch_layout(pairs, cl, split, Q.dump_bytes).total > scratch_bytes)) continue;
                    int per_sm = (228 * 1024) / (smem + 1024);
                    if (per_sm > kMaxCtasPerSm) per_sm = kMaxCtasPerSm;
                    if (per_sm < 1) continue;
                    const int n_warps = kAW * cl * split;
                    const int upw = ((P.tiles_total + n_warps - 1) / n_warps) * unit_tile + ((n_rt + n_warps - 1) / n_warps);
                    const double fixed = launches == 2 ? 4.0 + 0.05 * split : 3.0;
                    const double cost = plan_cost(pairs * cl * split, cl, per_sm, pair_units / n_warps, upw, fixed, ns);
                    if (cost < best_cost - 1e-9) { best_cost = cost; best_cl = cl; best_ns = ns; best_split = split; best_launches = launches; best_extra = -1; }
                }
            }
        }
    }
    // Uneven form: independent CTAs (cluster 1), as many as the GPU holds at once, nsplit or nsplit + 1 of them per pair.
    // Not with an exchange (the ranks' launches and a single-GPU launch of the same tensors must be able to share a plan)
    // and not when the caller forces a uniform plan.
    const bool forced_uniform = want_extra == 0 && (want_cl || want_split || want_launches);
    if (scratch && !xch && !forced_uniform && P.tiles_total > 0 && (want_launches == 0 || want_launches == 2)) {
        for (int per_sm = kMaxCtasPerSm; per_sm >= 1; per_sm--) {
            const long T = (long)kSmCount * per_sm;
            int base = (int)(T / pairs), extra = (int)(T % pairs);
            if (want_extra > 0) { base = want_split; extra = want_extra; }
            if (base < 1 || base + 1 > 128 || extra >= pairs) { if (want_extra > 0) break; continue; }
            if (extra == 0 && want_extra == 0) continue;      // a uniform plan: covered above
            bool found = false;
            for (int ns = 2; ns >= 1; ns--) {
                if (env_slots && ns != env_slots) continue;
                AttnDev Q = P;
                const int smem = plan_smem(Q, 1, base, ns, slot);
                if (smem > 227 * 1024) continue;
                if (scratch_layout(pairs, 1, base + 1, Q.dump_bytes).total > scratch_bytes) continue;
                int fit = (228 * 1024) / (smem + 1024);
                if (fit > kMaxCtasPerSm) fit = kMaxCtasPerSm;
                if (fit < per_sm && want_extra == 0) continue;
                const long ctas = pairs * base + extra;
                const int n_warps = kAW * base;
                const int upw = ((P.tiles_total + n_warps - 1) / n_warps) * unit_tile + ((n_rt + n_warps - 1) / n_warps);
                const double cost = plan_cost(ctas, 1, fit, pair_units * pairs / ((double)ctas * kAW), upw, 4.0 + 0.05 * (base + 1), ns);
                if (cost < best_cost - 1e-9 || want_extra > 0) {
                    best_cost = cost; best_cl = 1; best_ns = ns; best_split = base; best_launches = 2; best_extra = extra;
                    found = true;
                    if (want_extra > 0) break;
                }
            }
            if (found || want_extra > 0) break;               // the fullest GPU that fits is the candidate
        }
    }
    if (best_cl == 0) return kUnsupported;
    const int smem = plan_smem(P, best_cl, best_split, best_ns, slot);
    P.extra = best_extra;
    if (best_launches == 2) {
        const ScratchLayout L = scratch_layout(pairs, best_cl, best_extra >= 0 ? best_split + 1 : best_split, P.dump_bytes);
        if (!scratch || L.total > scratch_bytes) return kBadArgument;
        uint8_t* base = static_cast<uint8_t*>(scratch);
        P.sc_count = reinterpret_cast<unsigned*>(base + L.count);
        P.sc_ml = reinterpret_cast<float*>(base + L.ml);
        P.sc_part = reinterpret_cast<float*>(base + L.part);
        P.sc_scores = base + L.scores;
    }
    if (plan_io) { plan_io->cluster = best_cl; plan_io->nsplit = best_split; plan_io->launches = best_launches; plan_io->extra = best_extra > 0 ? best_extra : 0; }
    if (dry_run) return kOk;
    dim3 grid(P.cluster * P.nsplit, a.kv_heads, a.batch);
    if (best_extra >= 0) grid = dim3((unsigned)(pairs * best_split + best_extra), 1, 1);
    return a.is_bf16 ? launch_typed<__nv_bfloat16>(P, grid, smem, st) : launch_typed<__half>(P, grid, smem, st);
}

}  // namespace pkv
