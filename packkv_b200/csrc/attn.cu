// Fused decompress-attention decode for one query token per sequence.
//
// Replaces, in one launch over the packed streams, the reference's kq_mat_vec_mul + fused_kq
// (packkv_cuda_ext/src/kernels.cu:426-535, fused_kernels.cu:13-76), torch softmax
// (evaluation/evaluation.py:1040-1049), wv_mat_vec_mul + fused_wv (kernels.cu:632-765,
// fused_kernels.cu:187-261) and, for numerics, the model path's dequantise-then-attend
// (models/cache/packkv_quant.py:45-85 + models/llama.py:177-212).  Decompressed K/V never go
// to HBM, and neither do scores or partial results.
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
//   phase 1  every warp of the cluster walks its 128-token (or 64-token) tiles: K blocks are
//            staged with cp.async, unpacked, dequantised and contracted with q on the tensor
//            cores; scores stay in the warp's shared memory.  Residual (uncompressed) tokens
//            are 16-token tiles handed to the same warps and contracted by the same mma
//            (K rows straight from global memory as A fragments, V rows staged in shared
//            memory and transposed on load with ldmatrix).
//   exchange per-CTA (max, sum) go through distributed shared memory, one cluster barrier.
//   phase 2  scores -> probabilities in place, V blocks are unpacked and contracted.
//   reduce   warps -> CTA in shared memory, CTAs -> rank 0 through distributed shared memory.
//
// Per warp, K: read the per-round headers, warp-scan the pack sizes into byte offsets, unpack
// 4 channels x 16 tokens per lane with one rotate + one mask per code, exchange through a
// swizzled 16x128-byte tile so that each lane holds the mma A fragment (tokens x channels),
// dequantise two codes per instruction, mma.sync m16n8k16 against the q fragments (the 8
// columns of the n-tile are the q heads of the group).  V: same unpack (1 channel x 64 tokens
// per lane), 32x64-byte exchange tile, A = channels x tokens, B = probabilities.
#include <cooperative_groups.h>

#include "attn.cuh"
#include "common.cuh"

namespace cg = cooperative_groups;

namespace pkv {

constexpr int kAW = 4;            // warps per CTA
// staging slots per warp: 2 = the copy of the next block overlaps the work on this one; 1 = the next block is
// only prefetched to L2 (9 KB less shared memory per CTA, measured 5 % slower at the same 4 CTAs per SM; a fifth
// CTA would also need 96 registers per thread, which spills and is slower still)
constexpr int kSlots = 2;
constexpr int kCtasPerSm = 4;
constexpr int kD = 128;           // head dimension

// ---- element-type traits --------------------------------------------------------------------
template <typename T> struct Tr;

template <> struct Tr<__half> {
    using T2 = __half2;
    static constexpr unsigned kMagic = 0x64646464u;   // 0x6400 | b == 1024 + b, exact
    static constexpr float kBias = 1024.f;
    static __device__ __forceinline__ T2 bias2() { return __float2half2_rn(1024.f); }
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
    static constexpr unsigned kMagic = 0x43434343u;   // 0x4300 | b == 128 + b, exact
    static constexpr float kBias = 128.f;
    static __device__ __forceinline__ T2 bias2() { return __float2bfloat162_rn(128.f); }
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

// two biased codes (bias + code, exact) -> two dequantised elements, rounded like the reference
template <typename T, bool HP>
__device__ __forceinline__ unsigned deq2(unsigned biased, typename Tr<T>::T2 z, typename Tr<T>::T2 s) {
    using T2 = typename Tr<T>::T2;
    T2 x = as_t2<T2>(biased);
    if (!HP) return as_u(__hmul2(__hadd2(x, z), s));          // z = zero - bias
    // the product must be rounded before the addition, as in the reference: _rn keeps the compiler from
    // contracting the pair into one fused multiply-add
    return as_u(__hadd2(__hmul2_rn(__hsub2(x, Tr<T>::bias2()), s), z));   // z = min
}

__device__ __forceinline__ void cp_async16(uint8_t* smem_dst, const uint8_t* gsrc) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gsrc));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// exp(x) for x <= 0 (softmax arguments): one multiply and one MUFU; results below the normal
// range flush to zero, which the rounding to the element type does anyway
__device__ __forceinline__ float fast_exp(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
    return y;
}
__device__ __forceinline__ void cp_async16_zfill(unsigned smem_dst, const void* gsrc, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_dst), "l"(gsrc), "r"(valid ? 16 : 0));
}
// four 8x8 b16 matrices, transposed on load: lane l passes the address of row l%8 of matrix l/8
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned addr, unsigned (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}

// header fields of width w at bits 0, w, 2w, 3w of a lane word -> one byte each
struct FieldSpread { int s1, s2; unsigned m1, m2; };
__device__ __forceinline__ unsigned spread_fields(unsigned x, const FieldSpread& f) {
    const unsigned y = (x | (x << f.s1)) & f.m1;
    return (y | (y << f.s2)) & f.m2;
}
__host__ inline FieldSpread make_field_spread(int w) {
    return FieldSpread{16 - 2 * w, 8 - w, ((1u << (2 * w)) - 1u) * 0x00010001u, ((1u << w) - 1u) * 0x01010101u};
}

// One pack (16 codes of `len` bits, token 0 in the top bits of the 2*len-byte word) -> 16 bytes.
// la = {2^(4 len) - 1, (2^(2 len) - 1) * 0x00010001, (2^len - 1) * 0x01010101, 4 len},
// lb = {16 - 2 len, 8 - len, 8 len, -}: the table entry of this length.  Fields are spread by two
// shift-or-mask steps per four codes; byte p of the result holds token p ^ 3 (the consumers pick
// their byte pairs accordingly), each plus the pack minimum replicated in `minrep`.
__device__ __forceinline__ uint4 unpack_pack(unsigned lo, unsigned hi, const uint4& la, const uint4& lb, unsigned minrep) {
    const unsigned tp = __funnelshift_rc(lo, hi, lb.z);
    unsigned w[4] = {(tp >> la.w) & la.x, tp & la.x, (lo >> la.w) & la.x, lo & la.x};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const unsigned y = (w[i] | (w[i] << lb.x)) & la.y;
        w[i] = ((y | (y << lb.y)) & la.z) + minrep;
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ unsigned byte_of(unsigned x, int j) { return __byte_perm(x, 0, 0x4440 + j); }

// Channel order of the K contraction.  mma step j = 2m + b covers, for the lanes with c = lane & 3,
// the channels 32m + 8c + {2b, 2b+4} (k = 2c, 2c+1) and 32m + 8c + {2b+1, 2b+5} (k = 2c+8, 2c+9): the
// order in which ldmatrix.trans delivers the exchange tile.  From the 8 consecutive elements
// x0..x7 of channels 32m + 8c.. this forms the four operand registers of steps 2m and 2m+1:
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
    int prow;            // bytes of one row of the score / probability tile
    int warp_smem;       // bytes of per-warp shared memory
    int cta_off;         // byte offset of the CTA-shared block
    int out_off;         // byte offset, inside a warp's region, of its rows of the CTA's reduced output
    int tile_shift, cbk_shift, cbv_shift;   // log2 of tile, cbk, cbv
    int nkb_shift, nvi_shift;               // log2 of K blocks per tile and of V blocks (2 halves x token blocks) per tile
    FieldSpread klen, kmin, vlen, vmin;     // header field widths -> bytes
};

// CTA-shared block (cluster-visible)
struct CtaShared {
    float cl_m[8];       // this CTA's max per head
    float cl_l[8];       // this CTA's sum of exp(s - cl_m) per head
    float wm[kAW][8];    // per-warp scratch
    float gM[8], gInvL[8];
};
// The CTA's reduced accumulators out[head][channel] (read by rank 0 through distributed shared
// memory) live in the warps' exchange tiles, which are idle by then: head hd -> warp hd & 3,
// float offset (hd >> 2) * kD.
__device__ __forceinline__ float* cta_out_row(uint8_t* smem, int warp_smem, int out_off, int hd) {
    return reinterpret_cast<float*>(smem + (hd & 3) * warp_smem + out_off) + (hd >> 2) * kD;
}

// =================================================================================================
template <typename T, int KMODE, bool HP>
__global__ void __launch_bounds__(kAW * 32, kCtasPerSm) attn_decode_kernel(const AttnDev P) {
    using T2 = typename Tr<T>::T2;
    extern __shared__ __align__(16) uint8_t smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const AttnArgs& a = P.a;
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int rank = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int G = a.group;
    const int q_heads = a.kv_heads * G;
    const int n_warps = kAW * P.cluster;
    const int gw = rank * kAW + wic;                   // warp index inside the cluster

    uint8_t* wbase = smem + wic * P.warp_smem;
    uint8_t* xch = wbase + kSlots * P.slot;            // 2048 B exchange tile
    T* vsz = reinterpret_cast<T*>(xch + 2048);         // [tile] V scale, [tile] V zero(-bias)
    T* ksz = vsz + 2 * P.tile;                         // token mode: [tile] K scale, [tile] K zero(-bias)
    uint8_t* stile = reinterpret_cast<uint8_t*>(ksz + 2 * P.tile);   // [tpw][rows][prow] scores -> probabilities
    const unsigned rst_a = smem_addr(stile + P.tpw * P.rows * P.prow);      // [rtw][rows][16] residual scores -> probabilities
    CtaShared* cs = reinterpret_cast<CtaShared*>(smem + P.cta_off);
    // 32-bit shared-window addresses for the hot loops
    const unsigned wbase_a = smem_addr(wbase), xch_a = smem_addr(xch), vsz_a = smem_addr(vsz), stile_a = smem_addr(stile);
    // K exchange tile: one 16-byte row (16 tokens) per channel; channel 4*lane + i lives in row
    // lane + 32*i, so the four row stores of a warp are contiguous and the 8x8 matrices that
    // ldmatrix.trans turns into fragments (plane i, rows 8m..8m+7) are contiguous too.
    const unsigned kst = xch_a + lane * 16;
    const unsigned kldm = xch_a + (32 * (lane >> 3) + (lane & 7)) * 16;
    // V exchange: row = lane (channel), chunk swizzle by (row >> 1) & 3; fragment rows g, g+8, g+16, g+24 share that swizzle
    const unsigned vst = xch_a + lane * 64, vsw = ((lane >> 1) & 3) << 4;
    const unsigned vld = xch_a + g * 64 + ((c ^ ((g >> 1) & 3)) << 4);

    const int my_tiles = gw < P.tiles_total ? (P.tiles_total - gw + n_warps - 1) / n_warps : 0;
    // residual tiles are dealt from the last warp backwards (the compressed tiles are dealt from
    // the first warp forwards, so the warps with one tile fewer take them)
    const int n_rt = (a.n_res + 15) >> 4, rslot = n_warps - 1 - gw;
    const int my_rt = rslot < n_rt ? (n_rt - rslot + n_warps - 1) / n_warps : 0;
    const int nkb = 1 << P.nkb_shift, nvi = 1 << P.nvi_shift;   // K blocks / V blocks per tile
    const int k_items = my_tiles << P.nkb_shift, v_items = my_tiles << P.nvi_shift;
    const int total_items = k_items + v_items;
    const int k_rounds = a.cbk >> 4;
    const int lbk = len_field_bits(a.bits_k), lbv = len_field_bits(a.bits_v);
    const uint8_t* kbase = a.k_stream + (int64_t)b * a.k_seq_stride;
    const uint8_t* vbase = a.v_stream + (int64_t)b * a.v_seq_stride;
    const uint32_t* kinfo = a.k_info + (int64_t)b * a.k_info_seq_stride * 2;
    const uint32_t* vinfo = a.v_info + (int64_t)b * a.v_info_seq_stride * 2;
    const T2 bias2 = Tr<T>::bias2();
    const bool col_live = 2 * c < P.rows;              // this lane's score columns (heads 2c, 2c+1) are kept

    // ---- stream-block fetch ---------------------------------------------------------------------
    // item n < k_items: K block (n % nkb) of local tile n / nkb; else V block of local tile
    // (offset, size) of item n's block; loaded one item ahead of the copy that needs it
    auto load_info = [&](int n) -> uint2 {
        const uint32_t* info;
        if (n < k_items) {
            const int tl = n >> P.nkb_shift, i = n & (nkb - 1);
            const int t0 = (gw + tl * n_warps) << P.tile_shift;
            info = kinfo + ((int64_t)((t0 >> P.cbk_shift) + i) * a.kv_heads + h) * 2;
        } else {
            const int m = n - k_items;
            const int tl = m >> P.nvi_shift, vi = m & (nvi - 1);
            const int t0 = (gw + tl * n_warps) << P.tile_shift;
            info = vinfo + ((int64_t)((t0 >> P.cbv_shift) + (vi >> 1)) * (2 * a.kv_heads) + 2 * h + (vi & 1)) * 2;
        }
        return __ldg(reinterpret_cast<const uint2*>(info));
    };
    // Starts the copy of item n's block into its staging slot, together with the quantisation
    // parameters the item needs: channel-mode K: the block's 128 scales and 128 zero-points
    // (512 bytes at vsz, free during phase 1); first V block of a tile: the tile's per-token
    // scales and zero-points into parameter buffer (tile & 1) (vsz / ksz, both free in phase 2).
    auto issue = [&](int n, uint2 inf, int& phase_out, int& size_out) {
        const uint8_t* base;
        int64_t cap;
        int bound;
        if (n < k_items) {
            base = kbase; cap = a.k_capacity;
            bound = 2 * k_rounds + k_rounds * (16 * a.bits_k + 16 * lbk + 256 * a.bits_k);
            if (KMODE == kKChannel) {
                const int tl = n >> P.nkb_shift, i = n & (nkb - 1);
                const int t0 = (gw + tl * n_warps) << P.tile_shift;
                const int64_t row = ((int64_t)(b * a.kv_heads + h) * a.param_blocks + ((t0 >> P.cbk_shift) + i)) * kD;
                const T* src = reinterpret_cast<const T*>(lane < 16 ? a.k_scale : a.k_zero) + row + 8 * (lane & 15);
                cp_async16(reinterpret_cast<uint8_t*>(vsz) + 16 * lane, reinterpret_cast<const uint8_t*>(src));
            }
        } else {
            const int m = n - k_items;
            const int tl = m >> P.nvi_shift, vi = m & (nvi - 1);
            base = vbase; cap = a.v_capacity;
            const int nseg = a.cbv == 128 ? 4 : 2;
            bound = 2 * nseg + nseg * (16 * a.bits_v + 16 * lbv + 256 * a.bits_v);
            if (vi == 0) {
                const int t0 = (gw + tl * n_warps) << P.tile_shift;
                const int chunks = P.tile >> 3;              // 16-byte chunks per parameter array
                if (lane < 2 * chunks) {
                    const T* src = reinterpret_cast<const T*>(lane < chunks ? a.v_scale : a.v_zero) + (int64_t)b * a.param_tokens + t0 +
                                   8 * (lane < chunks ? lane : lane - chunks);
                    cp_async16(reinterpret_cast<uint8_t*>(vsz) + (tl & 1) * 4 * P.tile + 16 * lane, reinterpret_cast<const uint8_t*>(src));
                }
            }
        }
        const unsigned off = inf.x, size = inf.y;
        uint8_t* dst = wbase + (kSlots == 2 ? (n & 1) : 0) * P.slot;
        if ((int64_t)off + size > cap || (int)size > bound || size < 4 || ((off | size) & 1u)) {   // blocks start and end on even bytes
            if (lane == 0) atomicOr(a.flags, kFlagBadStream);
            phase_out = 0; size_out = 0;
        } else {
            const uint8_t* src = base + off;
            const int phase = (int)(reinterpret_cast<uintptr_t>(src) & 15);
            const int total = (phase + (int)size + 15) & ~15;
            for (int j = lane * 16; j < total; j += 512) cp_async16(dst + j, src - phase + j);
            phase_out = phase; size_out = (int)size;
        }
        cp_async_commit();
    };

    // with one slot the next block cannot be copied while this one is in use: it is pulled into L2 instead
    auto prefetch_l2 = [&](int n, uint2 inf2) {
        const uint8_t* src = (n < k_items ? kbase : vbase) + inf2.x;
        const int64_t cap = n < k_items ? a.k_capacity : a.v_capacity;
        if ((int64_t)inf2.x + inf2.y <= cap && inf2.y <= 8192u)
            for (unsigned j = lane * 128u; j < inf2.y; j += 4096u) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + j));
    };
    int cur_phase = 0, cur_size = 0, nxt_phase = 0, nxt_size = 0;
    uint2 inf = make_uint2(0, 0);
    if (total_items > 0) issue(0, load_info(0), nxt_phase, nxt_size);
    if (total_items > 1) inf = load_info(1);

    // unpack table: two 16-byte entries per pack length 0..4 (see unpack_pack)
    __shared__ uint4 ulut[10];
    if (threadIdx.x < 5) {
        const unsigned L = threadIdx.x;
        ulut[2 * L] = make_uint4(L == 4 ? 0xFFFFu : (1u << (4 * L)) - 1u, ((1u << (2 * L)) - 1u) * 0x00010001u, ((1u << L) - 1u) * 0x01010101u, 4 * L);
        ulut[2 * L + 1] = make_uint4(16 - 2 * L, 8 - L, 8 * L, 0);
    }
    const unsigned ulut_a = smem_addr(ulut);
    bool bad_len = false;
    __syncthreads();

    // q fragments: column g of the n-tile is q head g
    unsigned qf[8][2];
    {
        const uint4* qp = reinterpret_cast<const uint4*>(
            reinterpret_cast<const T*>(a.q) + ((int64_t)(b * q_heads + h * G + min(g, G - 1))) * kD + 8 * c);
#pragma unroll
        for (int m = 0; m < 4; m++) {
            const uint4 v = g < G ? __ldg(qp + 4 * m) : make_uint4(0, 0, 0, 0);
            pair_shuffle(v, qf[2 * m], qf[2 * m + 1]);
        }
    }

    float mloc0 = -INFINITY, mloc1 = -INFINITY;       // running max of this lane's scores, heads 2c and 2c+1

    // ============================================================================ phase 1: K tiles
    for (int n = 0; n < k_items; n++) {
        cur_phase = nxt_phase; cur_size = nxt_size;
        cp_async_wait<0>();
        __syncwarp();
        // channel mode: per-(block, channel) scale and zero of this lane's channels, in mma order
        T2 ksc[8][2], kzb[8][2];
        if (KMODE == kKChannel) {
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const uint4 sv = lds128(vsz_a + 64 * m + 16 * c), zv = lds128(vsz_a + 256 + 64 * m + 16 * c);
                unsigned s0[2], s1[2], z0[2], z1[2];
                pair_shuffle(sv, s0, s1);
                pair_shuffle(zv, z0, z1);
                ksc[2 * m][0] = as_t2<T2>(s0[0]); ksc[2 * m][1] = as_t2<T2>(s0[1]);
                ksc[2 * m + 1][0] = as_t2<T2>(s1[0]); ksc[2 * m + 1][1] = as_t2<T2>(s1[1]);
                kzb[2 * m][0] = as_t2<T2>(z0[0]); kzb[2 * m][1] = as_t2<T2>(z0[1]);
                kzb[2 * m + 1][0] = as_t2<T2>(z1[0]); kzb[2 * m + 1][1] = as_t2<T2>(z1[1]);
            }
            if (!HP) {
#pragma unroll
                for (int j = 0; j < 8; j++) { kzb[j][0] = __hsub2(kzb[j][0], bias2); kzb[j][1] = __hsub2(kzb[j][1], bias2); }
            }
            __syncwarp();                              // every lane has its parameters before the next copy lands
        }
        if (n + 1 < total_items) {
            if (kSlots == 2) {
                issue(n + 1, inf, nxt_phase, nxt_size);
                if (n + 2 < total_items) inf = load_info(n + 2);
            } else {
                prefetch_l2(n + 1, inf);
            }
        }
        const unsigned blk = wbase_a + (kSlots == 2 ? (n & 1) : 0) * P.slot + cur_phase;
        const int tl = n >> P.nkb_shift, i = n & (nkb - 1);
        const int t0 = (gw + tl * n_warps) << P.tile_shift;
        const unsigned st = stile_a + tl * P.rows * P.prow;

        if (KMODE == kKToken && i == 0) {
            const T* ks = reinterpret_cast<const T*>(a.k_scale) + (int64_t)b * a.param_tokens + t0;
            const T* kz = reinterpret_cast<const T*>(a.k_zero) + (int64_t)b * a.param_tokens + t0;
            for (int t = lane; t < P.tile; t += 32) {
                ksz[t] = ks[t];
                ksz[P.tile + t] = HP ? kz[t] : Tr<T>::from_float(Tr<T>::to_float(kz[t]) - Tr<T>::kBias);
            }
            __syncwarp();
        }
        if (cur_size > 0) {
            const int bits_k = a.bits_k;
            int pos = 2 * k_rounds;
            for (int r = 0; r < k_rounds; r++) {
                const unsigned hdr = blk + pos;
                const unsigned minword = lds_lane_field(hdr, lane, 4 * bits_k);
                const unsigned lenword = lds_lane_field(hdr + 16 * bits_k, lane, 4 * lbk);
                unsigned lens4 = spread_fields(lenword, P.klen);          // byte j = length of pack j
                const unsigned mins4 = spread_fields(minword, P.kmin);
                if ((lens4 + 0x03030303u) & 0x08080808u) { lens4 = 0; bad_len = true; }   // no encoder writes a length above 4
                const unsigned inc = warp_inclusive_sum(lens4);
                const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
                const unsigned exc = inc - lens4;
                const unsigned packs = hdr + 16 * bits_k + 16 * lbk;
                const unsigned lidx = lens4 << 5;                          // byte j = offset of the table entry
                unsigned before = 0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    unsigned lo, hi;
                    lds_u64_align2(packs + 2 * (before + byte_of(exc, j)), lo, hi);
                    before += byte_of(tot, j);
                    const unsigned le = ulut_a + byte_of(lidx, j);
                    const uint4 la = lds128(le), lb = lds128(le + 16);
                    sts128(kst + 512 * j, unpack_pack(lo, hi, la, lb, __byte_perm(mins4, 0, 0x1111 * j)));
                }
                __syncwarp();
                unsigned fr[4][4];
#pragma unroll
                for (int m = 0; m < 4; m++) ldmatrix_x4_trans(kldm + 128 * m, fr[m]);
                __syncwarp();
                // Lane (g, c) holds, per plane, channels (row 2c | row 2c+1) x tokens (2(g^1)+1 | 2(g^1)):
                // fragment row g is token T0 = 2(g^1), row g+8 is token T0 + 1.
                const int tk = i * a.cbk + r * 16 + 2 * (g ^ 1);
                T2 sg, zg, sg8, zg8;                         // token mode: per-row scale / zero
                if (KMODE == kKToken) {
                    const unsigned sv = lds32(smem_addr(ksz) + 2 * tk), zv = lds32(smem_addr(ksz) + 2 * (P.tile + tk));
                    sg = as_t2<T2>(__byte_perm(sv, sv, 0x1010)); sg8 = as_t2<T2>(__byte_perm(sv, sv, 0x3232));
                    zg = as_t2<T2>(__byte_perm(zv, zv, 0x1010)); zg8 = as_t2<T2>(__byte_perm(zv, zv, 0x3232));
                }
                float accs[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};   // two chains hide the mma latency
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const unsigned u0 = fr[j >> 1][2 * (j & 1)], u1 = fr[j >> 1][2 * (j & 1) + 1];
                    const unsigned a0 = __byte_perm(u0, Tr<T>::kMagic, 0x4341), a1 = __byte_perm(u0, Tr<T>::kMagic, 0x4240);
                    const unsigned a2 = __byte_perm(u1, Tr<T>::kMagic, 0x4341), a3 = __byte_perm(u1, Tr<T>::kMagic, 0x4240);
                    unsigned af[4];
                    if (KMODE == kKChannel) {
                        af[0] = deq2<T, HP>(a0, kzb[j][0], ksc[j][0]);
                        af[1] = deq2<T, HP>(a1, kzb[j][0], ksc[j][0]);
                        af[2] = deq2<T, HP>(a2, kzb[j][1], ksc[j][1]);
                        af[3] = deq2<T, HP>(a3, kzb[j][1], ksc[j][1]);
                    } else {
                        af[0] = deq2<T, HP>(a0, zg, sg);
                        af[1] = deq2<T, HP>(a1, zg8, sg8);
                        af[2] = deq2<T, HP>(a2, zg, sg);
                        af[3] = deq2<T, HP>(a3, zg8, sg8);
                    }
                    Tr<T>::mma(accs[j & 1], af, qf[j][0], qf[j][1]);
                }
                // scores rounded like the reference: matmul output, then * scaling; tokens T0, T0+1 share a store
                // (lanes whose head columns are not kept compute too: only the stores are predicated, no branch)
                {
                    const unsigned row0 = st + (2 * c) * P.prow + 2 * tk;
                    const unsigned p0 = Tr<T>::pack2(Tr<T>::round(accs[0][0] + accs[1][0]) * a.scaling, Tr<T>::round(accs[0][2] + accs[1][2]) * a.scaling);
                    const unsigned p1 = Tr<T>::pack2(Tr<T>::round(accs[0][1] + accs[1][1]) * a.scaling, Tr<T>::round(accs[0][3] + accs[1][3]) * a.scaling);
                    if (col_live) sts32(row0, p0);
                    if (col_live) sts32(row0 + P.prow, p1);
                    const float2 f0 = Tr<T>::unpack2(p0), f1 = Tr<T>::unpack2(p1);
                    mloc0 = fmaxf(mloc0, fmaxf(f0.x, f0.y));
                    mloc1 = fmaxf(mloc1, fmaxf(f1.x, f1.y));
                }
                pos += 16 * bits_k + 16 * lbk + 2 * (int)before;
            }
        }
        __syncwarp();
        if (kSlots == 1 && n + 1 < total_items) {
            issue(n + 1, inf, nxt_phase, nxt_size);
            if (n + 2 < total_items) inf = load_info(n + 2);
        }
    }

    // ---- residual tiles, phase 1: scores -------------------------------------------------------
    // A fragments come straight from the uncompressed rows: lane (g, c) reads channels
    // 32m + 8c .. +7 (m = 0..3) of tokens g and g+8 and pairs them in the order of the q fragments.
    const T* kres = reinterpret_cast<const T*>(a.k_res) + (int64_t)b * a.res_seq_stride + (int64_t)h * a.res_head_stride;
    const T* vres = reinterpret_cast<const T*>(a.v_res) + (int64_t)b * a.res_seq_stride + (int64_t)h * a.res_head_stride;
    for (int k = 0; k < my_rt; k++) {
        const int tok0 = (rslot + k * n_warps) << 4;
        const int ta = tok0 + g, tb = tok0 + g + 8;
        const uint4* pa = reinterpret_cast<const uint4*>(kres + (int64_t)min(ta, a.n_res - 1) * kD + 8 * c);
        const uint4* pb = reinterpret_cast<const uint4*>(kres + (int64_t)min(tb, a.n_res - 1) * kD + 8 * c);
        uint4 ra[4], rb[4];
#pragma unroll
        for (int m = 0; m < 4; m++) { ra[m] = __ldg(pa + 4 * m); rb[m] = __ldg(pb + 4 * m); }
        float accs[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int m = 0; m < 4; m++) {
            unsigned a0[2], a1[2], b0[2], b1[2];
            pair_shuffle(ra[m], a0, a1);
            pair_shuffle(rb[m], b0, b1);
            const unsigned f0[4] = {a0[0], b0[0], a0[1], b0[1]};
            const unsigned f1[4] = {a1[0], b1[0], a1[1], b1[1]};
            Tr<T>::mma(accs[0], f0, qf[2 * m][0], qf[2 * m][1]);
            Tr<T>::mma(accs[1], f1, qf[2 * m + 1][0], qf[2 * m + 1][1]);
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

    // ============================================================================ phase 2: V tiles
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) o[i][j] = 0.f;

    for (int n = k_items; n < total_items; n++) {
        cur_phase = nxt_phase; cur_size = nxt_size;
        cp_async_wait<0>();
        __syncwarp();
        if (n + 1 < total_items) {
            if (kSlots == 2) {
                issue(n + 1, inf, nxt_phase, nxt_size);
                if (n + 2 < total_items) inf = load_info(n + 2);
            } else {
                prefetch_l2(n + 1, inf);
            }
        }
        const unsigned blk = wbase_a + (kSlots == 2 ? (n & 1) : 0) * P.slot + cur_phase;
        const int m = n - k_items;
        const int tl = m >> P.nvi_shift, vi = m & (nvi - 1);
        const unsigned st_a = stile_a + tl * P.rows * P.prow;

        if (vi == 0) {
            // scores -> probabilities rounded to the element type, in place; V scale / zero of the tile
#pragma unroll
            for (int r = 0; r < 8; r++) {
                if (r < P.rows) {
                    const float M = cs->gM[r], I = cs->gInvL[r];
                    for (int ch = 0; ch < (P.tile >> 6); ch++) {
                        const unsigned ad = st_a + r * P.prow + 128 * ch + 4 * lane;
                        const float2 x = Tr<T>::unpack2(lds32(ad));
                        sts32(ad, Tr<T>::pack2(fast_exp(x.x - M) * I, fast_exp(x.y - M) * I));
                    }
                }
            }
            if (!HP) {
                // the tile's zero-points take the conversion bias once here instead of in every segment
                const unsigned zb = vsz_a + (tl & 1) * 4 * P.tile + 2 * P.tile;
                for (int t = lane; t < (P.tile >> 1); t += 32) sts32(zb + 4 * t, as_u(__hsub2(as_t2<T2>(lds32(zb + 4 * t)), bias2)));
            }
            __syncwarp();
        }
        if (cur_size > 0) {
            const int hh = vi & 1;                         // which 64-channel half of the head
            const int tok_blk = (vi >> 1) << P.cbv_shift;  // token offset of the block in the tile
            const int rpw_shift = a.cbv == 128 ? 1 : 0;
            const int nseg = 2 << rpw_shift;
            const int bits_v = a.bits_v;
            int pos = 2 * nseg;
            for (int sgi = 0; sgi < nseg; sgi++) {
                const int w = sgi >> rpw_shift, rr = sgi & ((1 << rpw_shift) - 1);
                const int tok_seg = tok_blk + rr * 64;     // first token (in the tile) of the segment
                const unsigned hdr = blk + pos;
                const unsigned minword = lds_lane_field(hdr, lane, 4 * bits_v);
                const unsigned lenword = lds_lane_field(hdr + 16 * bits_v, lane, 4 * lbv);
                unsigned lens4 = spread_fields(lenword, P.vlen);          // byte q = length of pack q (tokens 16q..16q+15)
                const unsigned mins4 = spread_fields(minword, P.vmin);
                if ((lens4 + 0x03030303u) & 0x08080808u) { lens4 = 0; bad_len = true; }
                const unsigned inc = warp_inclusive_sum(lens4);
                const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
                const unsigned exc = inc - lens4;
                const unsigned packs = hdr + 16 * bits_v + 16 * lbv;
                const unsigned lidx = lens4 << 5;
                unsigned before = 0;
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) {
                    unsigned lo, hi;
                    lds_u64_align2(packs + 2 * (before + byte_of(exc, q4)), lo, hi);
                    before += byte_of(tot, q4);
                    const unsigned le = ulut_a + byte_of(lidx, q4);
                    const uint4 la = lds128(le), lb = lds128(le + 16);
                    // row = lane (channel), logical 16-byte chunk q4, swizzled; byte p of the chunk is token 16*q4 + (p ^ 3)
                    sts128(vst + ((q4 << 4) ^ vsw), unpack_pack(lo, hi, la, lb, __byte_perm(mins4, 0, 0x1111 * q4)));
                }
                __syncwarp();
                // per-token scale / zero pairs and probabilities for tokens tok_seg + 16c .. +15
                const unsigned tok2 = 2 * (tok_seg + 16 * c);      // byte offset of this lane's 16 tokens in a row of halves
                const unsigned vpar = vsz_a + (tl & 1) * 4 * P.tile + tok2;   // this tile's parameter buffer
                const uint4 s0 = lds128(vpar), s1 = lds128(vpar + 16);
                const uint4 z0 = lds128(vpar + 2 * P.tile), z1 = lds128(vpar + 2 * P.tile + 16);
                // head columns beyond the kept rows read a kept row: their output columns are never used
                const unsigned prow_a = st_a + min(g, P.rows - 1) * P.prow + tok2;
                const uint4 p0 = lds128(prow_a), p1 = lds128(prow_a + 16);
                const unsigned vS[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                const unsigned vZ[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
                const unsigned pf[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
                // A fragments for both 16-channel row tiles, then the contraction into the
                // accumulator group of this (64-channel half, warp half): static register
                // indices, so the select is unrolled
                unsigned afr[2][4][4];
#pragma unroll
                for (int mt = 0; mt < 2; mt++) {
                    const uint4 xa = lds128(vld + (16 * mt) * 64), xb = lds128(vld + (16 * mt + 8) * 64);
                    const unsigned ua[4] = {xa.x, xa.y, xa.z, xa.w};
                    const unsigned ub[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        // bytes of a word are tokens 4j+3, 4j+2, 4j+1, 4j
                        afr[mt][j][0] = deq2<T, HP>(__byte_perm(ua[j], Tr<T>::kMagic, 0x4243), as_t2<T2>(vZ[2 * j]), as_t2<T2>(vS[2 * j]));
                        afr[mt][j][1] = deq2<T, HP>(__byte_perm(ub[j], Tr<T>::kMagic, 0x4243), as_t2<T2>(vZ[2 * j]), as_t2<T2>(vS[2 * j]));
                        afr[mt][j][2] = deq2<T, HP>(__byte_perm(ua[j], Tr<T>::kMagic, 0x4041), as_t2<T2>(vZ[2 * j + 1]), as_t2<T2>(vS[2 * j + 1]));
                        afr[mt][j][3] = deq2<T, HP>(__byte_perm(ub[j], Tr<T>::kMagic, 0x4041), as_t2<T2>(vZ[2 * j + 1]), as_t2<T2>(vS[2 * j + 1]));
                    }
                }
                const int sel = 2 * hh + w;
#pragma unroll
                for (int idx = 0; idx < 4; idx++) {
                    if (idx == sel) {
#pragma unroll
                        for (int mt = 0; mt < 2; mt++)
#pragma unroll
                            for (int j = 0; j < 4; j++) Tr<T>::mma(o[2 * idx + mt], afr[mt][j], pf[2 * j], pf[2 * j + 1]);
                    }
                }
                __syncwarp();
                pos += 16 * bits_v + 16 * lbv + 2 * (int)before;
            }
        }
        __syncwarp();
        if (kSlots == 1 && n + 1 < total_items) {
            issue(n + 1, inf, nxt_phase, nxt_size);
            if (n + 2 < total_items) inf = load_info(n + 2);
        }
    }
    cp_async_wait<0>();
    __syncwarp();
    if (__any_sync(0xffffffffu, bad_len) && lane == 0) atomicOr(a.flags, kFlagBadStream);

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
    {
        const int d = threadIdx.x;
        for (int hd = 0; hd < G; hd++) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kAW; w++) v += reinterpret_cast<const float*>(smem + w * P.warp_smem)[hd * kD + d];
            cta_out_row(smem, P.warp_smem, P.out_off, hd)[d] = v;
        }
    }
    cluster.sync();
    if (rank == 0) {
        const int d = threadIdx.x;
        for (int hd = 0; hd < G; hd++) {
            float v = 0.f;
            for (int r = 0; r < P.cluster; r++) v += cluster.map_shared_rank(cta_out_row(smem, P.warp_smem, P.out_off, hd), r)[d];
            reinterpret_cast<T*>(a.out)[((int64_t)(b * q_heads + h * G + hd)) * kD + d] = Tr<T>::from_float(v);
        }
    }
    cluster.sync();   // keep every CTA's shared memory alive until rank 0 has read it
}

// =================================================================================================
static int k_bound(int cb, int bits) { int r = cb / 16; return 2 * r + r * (16 * bits + 16 * len_field_bits(bits) + 256 * bits); }
static int v_bound(int cb, int bits) { int n = cb == 128 ? 4 : 2; return 2 * n + n * (16 * bits + 16 * len_field_bits(bits) + 256 * bits); }

template <typename T, int KM, bool HPV>
static int launch_one(const AttnDev& P, dim3 grid, int smem, cudaStream_t st) {
    auto kern = attn_decode_kernel<T, KM, HPV>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kCudaError;
    if (P.cluster > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) return kCudaError;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kAW * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = P.cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, P) == cudaSuccess ? kOk : kCudaError;
}

template <typename T>
static int launch_typed(const AttnDev& P, dim3 grid, int smem, cudaStream_t st) {
    const AttnArgs& a = P.a;
    if (a.k_mode == kKChannel) return a.high_precision_zero ? launch_one<T, kKChannel, true>(P, grid, smem, st) : launch_one<T, kKChannel, false>(P, grid, smem, st);
    return a.high_precision_zero ? launch_one<T, kKToken, true>(P, grid, smem, st) : launch_one<T, kKToken, false>(P, grid, smem, st);
}

int launch_attention(const AttnArgs& a, cudaStream_t st) {
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
    P.a = a;
    P.tile = (a.n_comp > 0 && (a.cbk == 128 || a.cbv == 128)) ? 128 : 64;
    P.tiles_total = a.n_comp / P.tile;
    auto lg2 = [](int v) { int s = 0; while ((1 << s) < v) s++; return s; };
    P.tile_shift = lg2(P.tile);
    P.cbk_shift = a.n_comp > 0 ? lg2(a.cbk) : 6;
    P.cbv_shift = a.n_comp > 0 ? lg2(a.cbv) : 6;
    P.nkb_shift = P.tile_shift - P.cbk_shift;
    P.nvi_shift = P.tile_shift - P.cbv_shift + 1;
    if (a.n_comp > 0) {
        P.klen = make_field_spread(len_field_bits(a.bits_k)); P.kmin = make_field_spread(a.bits_k);
        P.vlen = make_field_spread(len_field_bits(a.bits_v)); P.vmin = make_field_spread(a.bits_v);
    }
    // cluster size: enough CTAs for ~2 waves of the 148 SMs (3 CTAs each), but at least one
    // tile per warp; a long sequence must also fit its scores in shared memory
    const long pairs = (long)a.batch * a.kv_heads;
    const int units = P.tiles_total + (a.n_res + 15) / 16;
    int cl = 1;
    while (cl < 8 && pairs * cl < 2L * 148 * 3 && units > kAW * cl) cl *= 2;
    P.rows = (a.group + 1) & ~1;
    P.prow = 2 * P.tile + 16;
    int slot = 0;
    if (a.n_comp > 0) {
        const int kb = k_bound(a.cbk, a.bits_k), vb = v_bound(a.cbv, a.bits_v);
        slot = ((kb > vb ? kb : vb) + 48 + 15) & ~15;
    }
    if (a.n_res > 0 && kSlots * slot < 16 * 272) slot = 16 * 272 / kSlots;   // the residual V tile borrows the staging slots
    P.slot = slot;
    int smem = 0;
    for (;;) {
        P.cluster = cl;
        const int n_warps = kAW * cl;
        P.tpw = (P.tiles_total + n_warps - 1) / n_warps;
        P.rtw = ((a.n_res + 15) / 16 + n_warps - 1) / n_warps;
        int warp_smem = kSlots * slot + 2048 + 8 * P.tile + P.tpw * P.rows * P.prow + P.rtw * P.rows * 32;
        P.out_off = kSlots * slot > 8 * kD * 4 ? kSlots * slot : 8 * kD * 4;   // behind the parked accumulators
        const int red_need = P.out_off + 2 * kD * 4;
        if (warp_smem < red_need) warp_smem = red_need;
        P.warp_smem = (warp_smem + 15) & ~15;
        P.cta_off = kAW * P.warp_smem;
        smem = P.cta_off + (int)sizeof(CtaShared);
        if (smem <= 200 * 1024 || cl >= 16) break;
        cl *= 2;                                          // long sequence: spread the scores over more CTAs
    }
    if (smem > 227 * 1024) return kUnsupported;
    dim3 grid(P.cluster, a.kv_heads, a.batch);
    return a.is_bf16 ? launch_typed<__nv_bfloat16>(P, grid, smem, st) : launch_typed<__half>(P, grid, smem, st);
}

}  // namespace pkv
