// Single-pass encoder: fp16/bf16 K or V -> packed stream blocks, without a code matrix in HBM.
//
// Replaces, for the north-star pairing (K per-channel, V per-token), the reference's
// quant_ints (torch, utils/compute.py:84-112) + k/v_encode_cpu (C++ on the host,
// packkv_cuda_ext/src/{k,v}_encode_cpu.cpp); codes, parameters and block bytes are identical to
// the separate quantise + pack kernels.
//
// The stream format lays blocks back to back, so a block's byte offset is the sum of all earlier
// block sizes of its sequence.  Two forms:
//   direct : ONE launch.  A CTA builds its blocks (consecutive in the stream) in shared memory, then
//            learns the offset of its first block from the CTAs before it in the sequence by a
//            decoupled look-back over a small status array (every CTA publishes the bytes of its own
//            blocks as soon as it knows them, so nobody waits for more than its neighbours' packing),
//            and writes the blocks to their final place.  CTAs take their position from a ticket
//            counter, so every CTA a look-back waits for has started; the wait is bounded all the same
//            and a CTA that gives up raises the timeout flag and writes nothing.
//            HBM traffic per element: 2 B read (the second read of a tile comes from L1/L2) + the
//            block bytes written once (~0.56 B at 4 bit).
//   slots  : three launches, no device-side waiting (more than 8 heads, or on request): encode into
//            fixed-stride SLOTS in scratch memory with the size in block_info[blk][1]; per-sequence
//            exclusive scan (scan_sizes_kernel, pack.cu); one warp per block copies its slot to its
//            final offset.  The block bytes are written, read and written once more.
#include <cstdlib>
#include <string>

#include "common.cuh"
#include "launch.h"
#include "pack_dev.cuh"
#include "quant_dev.cuh"

namespace pkv {

struct FusedArgs {
    const void* x; int64_t sb, sh, ss;      // (B, H, S, 128), strides in elements
    void* scale; void* zero;
    int param_blocks, first_block;          // K channel mode parameter layout
    int param_tokens, first_token;          // V token mode parameter layout
    uint8_t* slots; int slot_stride;        // scratch: one slot per block, sequence-major
    uint32_t* info; int64_t info_seq_stride; int first_cb;
    int batch, heads, tokens, cb, bits;
    float rel;
    unsigned* flags;
    const uint8_t* order;                   // optional (batch, tokens / order_block, order_block): source row of every stored row
    int order_block;                        // tokens per reorder block (divides cb)
    // direct form (status != nullptr): blocks go straight to the stream
    unsigned* ticket;                       // zero before the launch: CTAs take their place in (sequence, link) order from it
    unsigned long long* status;             // [batch][links], zero before the launch: (state << 32) | bytes; state 1: this link's
                                            // blocks, 2: everything up to and including this link
    int links;                              // CTAs per sequence
    uint8_t* stream; int64_t stream_seq_stride, capacity;
    unsigned* stream_bytes;                 // per sequence: bytes in the stream before (in) and after (out) the call
};

#ifdef PKV_DEBUG_CHAIN
__device__ unsigned long long g_chain_stats[4];   // look-back cycles, look-backs, CTA cycles, CTAs
#endif
constexpr unsigned kChainSpins = 1u << 24;  // polls of a look-back before it gives up (each sleeps ~50 ns and waits for a load)

// The CTA's place in the launch: ticket t -> (sequence, link).  All threads call; one barrier.
__device__ __forceinline__ void chain_place(const FusedArgs& a, unsigned* sh_word, int& b, int& link) {
    if (threadIdx.x == 0) *sh_word = atomicAdd(a.ticket, 1u);
    __syncthreads();
    // sequences take turns: the links of one sequence that are in flight at the same time are few, so a look-back
    // rarely meets a predecessor that is still packing
    const unsigned t = *sh_word;
    b = (int)(t % (unsigned)a.batch);
    link = (int)(t / (unsigned)a.batch);
}

// Byte offset, in sequence b's stream, of the first block of link `link`, whose blocks hold `total` bytes in all.
// Called by ONE warp.  Returns false if a predecessor never published (bounded wait ran out).
__device__ __forceinline__ bool chain_offset(const FusedArgs& a, int b, int link, unsigned total, unsigned& offset) {
    const int lane = lane_id();
    unsigned long long* st = a.status + (int64_t)b * a.links;
    const unsigned base0 = a.first_cb == 0 ? 0u : a.stream_bytes[b];
    unsigned excl = 0;
    bool ok = true;
#ifdef PKV_DEBUG_CHAIN   // measurement builds: cycles and polls spent in look-backs
    const long long t_begin = clock64();
#endif
    if (link == 0) {
        excl = base0;
    } else {
        if (lane == 0) *reinterpret_cast<volatile unsigned long long*>(st + link) = (1ull << 32) | total;
        int j = link - 1;
        unsigned spins = 0;
        while (true) {
            const int idx = j - lane;
            const unsigned long long v = idx >= 0 ? *reinterpret_cast<volatile unsigned long long*>(st + idx) : ((2ull << 32) | base0);
            // the nearest link that knows everything before it ends the search; the links between it and this one
            // must have published their own bytes
            const unsigned done = __ballot_sync(0xffffffffu, (v >> 32) == 2);
            const int k = done ? __ffs(done) - 1 : 31;
            if (__any_sync(0xffffffffu, lane <= k && (v >> 32) == 0)) {
                if (++spins > kChainSpins) { ok = false; break; }
                __nanosleep(50);
                continue;
            }
            unsigned part = lane <= k ? (unsigned)v : 0u;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(0xffffffffu, part, d);
            excl += part;
            if (done) break;
            j -= 32;
        }
    }
#ifdef PKV_DEBUG_CHAIN
    if (lane == 0) {
        atomicAdd(&g_chain_stats[0], (unsigned long long)(clock64() - t_begin));
        atomicAdd(&g_chain_stats[1], 1ull);
    }
#endif
    // successors must not hang on a link that gave up: it publishes its own bytes on top of what it has
    if (lane == 0) {
        *reinterpret_cast<volatile unsigned long long*>(st + link) = (2ull << 32) | (excl + total);
        if (link == a.links - 1) a.stream_bytes[b] = excl + total;
        if (!ok) atomicOr(a.flags, kFlagTimeout);
    }
    offset = excl;
    return ok;
}

// One warp copies a finished block from shared memory (16-byte aligned) to its place in the stream (even address).
__device__ __forceinline__ void store_block(uint8_t* dst, const uint8_t* stage, int size, int lane) {
    const int phase = (int)(reinterpret_cast<uintptr_t>(dst) & 15);   // even
    const int head = min((16 - phase) & 15, size);                    // bytes before the first aligned chunk
    for (int j = 2 * lane; j < head; j += 64) *reinterpret_cast<uint16_t*>(dst + j) = *reinterpret_cast<const uint16_t*>(stage + j);
    const int nfull = (size - head) >> 4;
    const unsigned* s32 = reinterpret_cast<const unsigned*>(stage);
    const int sw = head >> 2;                                          // first source word of the body
    const unsigned sh = (unsigned)(head & 3) * 8;                      // 0 or 16: byte offset inside that word
    for (int c = lane; c < nfull; c += 32) {
        const unsigned* p = s32 + sw + 4 * c;                          // aligned 32-bit loads, realigned by funnel shifts
        const unsigned w0 = p[0], w1 = p[1], w2 = p[2], w3 = p[3], w4 = sh ? p[4] : 0u;
        *reinterpret_cast<uint4*>(dst + head + 16 * c) = make_uint4(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh),
                                                                    __funnelshift_r(w2, w3, sh), __funnelshift_r(w3, w4, sh));
    }
    for (int j = head + 16 * nfull + 2 * lane; j < size; j += 64)
        *reinterpret_cast<uint16_t*>(dst + j) = *reinterpret_cast<const uint16_t*>(stage + j);
}

// Direct form, after every warp of the CTA has put the sizes of its blocks into sizes[0..n): warp 0 gets the
// CTA's offset, then warp w stores the blocks w, w + nwarps, ... (block j at stage_of(j)) and their table entries.
// info_first: table index of block 0 of this link.  All threads call.
template <typename StageOf>
__device__ __forceinline__ void chain_store(const FusedArgs& a, int b, int link, const unsigned* sizes, int n, unsigned* sh_word, int64_t info_first,
                                            int nwarps, StageOf stage_of) {
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    __syncthreads();
    if (wic == 0) {
        unsigned total = 0;
        for (int j = 0; j < n; j++) total += sizes[j];
        unsigned off;
        const bool ok = chain_offset(a, b, link, total, off);
        if (lane == 0) *sh_word = ok ? off : 0xFFFFFFFFu;
    }
    __syncthreads();
    const unsigned base = *sh_word;
    if (base == 0xFFFFFFFFu) return;
    for (int j = wic; j < n; j += nwarps) {
        unsigned off = base;
        for (int i = 0; i < j; i++) off += sizes[i];
        const unsigned size = sizes[j];
        uint32_t* bi = a.info + ((int64_t)b * a.info_seq_stride + info_first + j) * 2;
        if (lane == 0) { bi[0] = off; bi[1] = size; }
        if ((int64_t)off + size > a.capacity) {
            if (lane == 0) atomicOr(a.flags, kFlagStreamOverflow);
            continue;
        }
        store_block(a.stream + (int64_t)b * a.stream_seq_stride + off, stage_of(j), (int)size, lane);
    }
}

__device__ __forceinline__ void store_slot(uint8_t* slot, const uint8_t* stage, int size, int lane) {
    // slot and stage are 16-byte aligned; the slot has room for the rounded-up size
    for (int i = 16 * lane; i < size; i += 512) *reinterpret_cast<uint4*>(slot + i) = *reinterpret_cast<const uint4*>(stage + i);
}

// ------------------------------------------------------------------------------------------ K
// rounds of one K block: quantise 16 tokens x 4 channels per lane, pack, append to `stage`
// ORDERED: stored row t of the block is source row ordp[t] (16-byte aligned table of the block's rows)
template <typename T, bool HP, int BITS, bool FAST, bool ORDERED>
__device__ __forceinline__ int k_encode_rounds(const T* x, int64_t ss, const uint8_t* ordp, const Quantiser<T, HP>& q0, const Quantiser<T, HP>& q1,
                                               const Quantiser<T, HP>& q2, const Quantiser<T, HP>& q3, const KGeom& g, uint8_t* stage,
                                               int lane, bool& bad) {
    constexpr int LB = len_field_bits(BITS);
    const int z0 = (int)q0.zero, z1 = (int)q1.zero, z2 = (int)q2.zero, z3 = (int)q3.zero;
    int pos = g.head_bytes;
    unsigned round_end = 0, over = 0;
    for (int r = 0; r < g.rounds; r++) {
        unsigned u[16];                               // four channel codes per token, one byte each
        unsigned mnj[4] = {255u, 255u, 255u, 255u}, mxj[4] = {0u, 0u, 0u, 0u};
        uint4 ob = make_uint4(0, 0, 0, 0);
        if (ORDERED) ob = __ldg(reinterpret_cast<const uint4*>(ordp + 16 * r));
        const unsigned ow[4] = {ob.x, ob.y, ob.z, ob.w};
#pragma unroll
        for (int t = 0; t < 16; t++) {
            const int row = ORDERED ? (int)((ow[t >> 2] >> (8 * (t & 3))) & 0xFFu) : r * 16 + t;
            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(x + (int64_t)row * ss));
            const T* e = reinterpret_cast<const T*>(&raw);
            const unsigned c0 = q0.template code_u8<FAST>(QT<T>::ld(e), z0), c1 = q1.template code_u8<FAST>(QT<T>::ld(e + 1), z1);
            const unsigned c2 = q2.template code_u8<FAST>(QT<T>::ld(e + 2), z2), c3 = q3.template code_u8<FAST>(QT<T>::ld(e + 3), z3);
            mnj[0] = min(mnj[0], c0); mxj[0] = max(mxj[0], c0);
            mnj[1] = min(mnj[1], c1); mxj[1] = max(mxj[1], c1);
            mnj[2] = min(mnj[2], c2); mxj[2] = max(mxj[2], c2);
            mnj[3] = min(mnj[3], c3); mxj[3] = max(mxj[3], c3);
            u[t] = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
        }
        unsigned minword = 0, lenword = 0, lens4 = 0;
        int len[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            over |= mxj[j] >> BITS;
            len[j] = min(bit_length_u32(mxj[j] - mnj[j]), BITS);
            minword |= (mnj[j] & ((1u << BITS) - 1u)) << (j * BITS);
            lenword |= (unsigned)len[j] << (j * LB);
            lens4 |= (unsigned)len[j] << (8 * j);
        }
        store_lane_fields_w<4 * BITS>(stage + pos, lane, minword);
        store_lane_fields_w<4 * LB>(stage + pos + g.min_bytes, lane, lenword);
        const unsigned inc = warp_inclusive_sum(lens4);
        const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
        const unsigned exc = inc - lens4;
        uint8_t* packs = stage + pos + g.min_bytes + g.len_bytes;
        unsigned before = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // tokens 0..7 and 8..15 as two words of at most 32 bits: w = w * 2^len + code, then the
            // minimum is taken off all eight fields at once (min * (1 + 2^len + ... + 2^(7 len)))
            const unsigned step = 1u << len[j];
            unsigned wt = 0, wb = 0, ones = 0;
#pragma unroll
            for (int t = 0; t < 8; t++) {
                wt = wt * step + __byte_perm(u[t], 0, 0x4440 + j);
                wb = wb * step + __byte_perm(u[t + 8], 0, 0x4440 + j);
                ones = ones * step + 1u;
            }
            wt -= mnj[j] * ones;
            wb -= mnj[j] * ones;
            const uint64_t w = ((uint64_t)wt << (8 * len[j])) | wb;
            store_pack_smem(packs + 2 * (before + ((exc >> (8 * j)) & 0xFFu)), w, len[j]);
            before += (tot >> (8 * j)) & 0xFFu;
        }
        const unsigned round_size = g.min_bytes + g.len_bytes + 2 * before;
        round_end += round_size;
        if (lane == 0) *reinterpret_cast<uint16_t*>(stage + 2 * r) = (uint16_t)round_end;
        pos += round_size;
    }
    bad = bad || over != 0;
    return pos;
}

// The same rounds for blocks whose four quantisers are packable(): two channels per instruction
// from the conversion to the pack minimum / maximum (16-bit lanes), then one multiply-add per code
// into the pack words.
template <typename T, int BITS, bool HALF, bool ORDERED>
__device__ __forceinline__ int k_encode_rounds_packed(const T* x, int64_t ss, const uint8_t* ordp, const Quantiser<T, false>& q0, const Quantiser<T, false>& q1,
                                                      const Quantiser<T, false>& q2, const Quantiser<T, false>& q3, const KGeom& g,
                                                      uint8_t* stage, int lane, bool& bad) {
    constexpr int LB = len_field_bits(BITS);
    const unsigned k01 = packed_code_bias(q0, q1), k23 = packed_code_bias(q2, q3);
    const HalfQuotient<T> h01(q0, q1), h23(q2, q3);      // used when every quantiser is in the half domain
    int pos = g.head_bytes;
    unsigned round_end = 0, over = 0;
    for (int r = 0; r < g.rounds; r++) {
        unsigned c01[16], c23[16];
        unsigned mn01 = 0xFFFFFFFFu, mx01 = 0u, mn23 = 0xFFFFFFFFu, mx23 = 0u;
        uint4 ob = make_uint4(0, 0, 0, 0);
        if (ORDERED) ob = __ldg(reinterpret_cast<const uint4*>(ordp + 16 * r));
        const unsigned ow[4] = {ob.x, ob.y, ob.z, ob.w};
#pragma unroll
        for (int t = 0; t < 16; t++) {
            const int row = ORDERED ? (int)((ow[t >> 2] >> (8 * (t & 3))) & 0xFFu) : r * 16 + t;
            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(x + (int64_t)row * ss));
            c01[t] = HALF ? h01.codes(raw.x) : packed_codes<T>(raw.x, q0, q1, k01);
            c23[t] = HALF ? h23.codes(raw.y) : packed_codes<T>(raw.y, q2, q3, k23);
            mn01 = min_u16x2(mn01, c01[t]); mx01 = max_u16x2(mx01, c01[t]);
            mn23 = min_u16x2(mn23, c23[t]); mx23 = max_u16x2(mx23, c23[t]);
        }
        over |= mx01 | mx23;
        const unsigned mnj[4] = {mn01 & 0xFFFFu, mn01 >> 16, mn23 & 0xFFFFu, mn23 >> 16};
        const unsigned d01 = mx01 - mn01, d23 = mx23 - mn23;     // lane-wise: no borrow, max >= min
        const unsigned dj[4] = {d01 & 0xFFFFu, d01 >> 16, d23 & 0xFFFFu, d23 >> 16};
        unsigned minword = 0, lenword = 0, lens4 = 0;
        int len[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            len[j] = min(bit_length_u32(dj[j]), BITS);
            minword |= (mnj[j] & ((1u << BITS) - 1u)) << (j * BITS);
            lenword |= (unsigned)len[j] << (j * LB);
            lens4 |= (unsigned)len[j] << (8 * j);
        }
        store_lane_fields_w<4 * BITS>(stage + pos, lane, minword);
        store_lane_fields_w<4 * LB>(stage + pos + g.min_bytes, lane, lenword);
        const unsigned inc = warp_inclusive_sum(lens4);
        const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
        const unsigned exc = inc - lens4;
        uint8_t* packs = stage + pos + g.min_bytes + g.len_bytes;
        unsigned before = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const unsigned step = 1u << len[j];
            unsigned wt = 0, wb = 0, ones = 0;
#pragma unroll
            for (int t = 0; t < 8; t++) {
                const unsigned ct = j < 2 ? c01[t] : c23[t], cb = j < 2 ? c01[t + 8] : c23[t + 8];
                wt = wt * step + ((j & 1) ? ct >> 16 : ct & 0xFFFFu);
                wb = wb * step + ((j & 1) ? cb >> 16 : cb & 0xFFFFu);
                ones = ones * step + 1u;
            }
            wt -= mnj[j] * ones;
            wb -= mnj[j] * ones;
            const uint64_t w = ((uint64_t)wt << (8 * len[j])) | wb;
            store_pack_smem(packs + 2 * (before + ((exc >> (8 * j)) & 0xFFu)), w, len[j]);
            before += (tot >> (8 * j)) & 0xFFu;
        }
        const unsigned round_size = g.min_bytes + g.len_bytes + 2 * before;
        round_end += round_size;
        if (lane == 0) *reinterpret_cast<uint16_t*>(stage + 2 * r) = (uint16_t)round_end;
        pos += round_size;
    }
    bad = bad || (over & ~(((1u << BITS) - 1u) * 0x00010001u)) != 0;
    return pos;
}

// one warp per K block (cb tokens x 128 channels of one head); lane owns channels 4l..4l+3, the
// same ownership as the stream format, so per-channel statistics need no cross-lane step.
// CONTIG: token rows are 128 elements apart (a contiguous (B, H, S, 128) tensor), so every load of a
// round is the block pointer plus a constant
#ifndef PKV_K_WARPS
#define PKV_K_WARPS 4
#endif
constexpr int kKWarps = PKV_K_WARPS;   // warps (= consecutive blocks of a sequence's stream) per CTA of the channel-mode K kernel
template <typename T, bool CONTIG, int BITS, bool ORDERED = false>
__global__ void __launch_bounds__(kKWarps * 32, 768 / (kKWarps * 32)) k_fused_encode_kernel(FusedArgs a) {
    constexpr bool HP = false;
    const int64_t ss = CONTIG ? 128 : a.ss;
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int LB = len_field_bits(BITS);
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    const int nctx = a.tokens / a.cb;
    const int64_t per_seq = (int64_t)nctx * a.heads;
    __shared__ unsigned sh_word, sh_sizes[kKWarps];
    const bool direct = a.status != nullptr;
    int b, rem, link = 0;
    int64_t warp = 0;
    if (direct) {
        // the CTA's warps take kKWarps consecutive blocks of one sequence's stream
        chain_place(a, &sh_word, b, link);
        rem = link * kKWarps + wic;
    } else {
        warp = (int64_t)blockIdx.x * kKWarps + wic;
        if (warp >= per_seq * a.batch) return;
        b = (int)(warp / per_seq);
        rem = (int)(warp % per_seq);
    }
    const bool active = rem < per_seq;
    const int cbi = active ? rem / a.heads : 0, h = active ? rem % a.heads : 0;
    const KGeom g(a.cb, BITS);
    const int slot_smem = (g.head_bytes + g.rounds * (g.min_bytes + g.len_bytes + 128 * 2 * BITS) + 15) & ~15;
    uint8_t* stage = smem + wic * slot_smem;
    const T* x = reinterpret_cast<const T*>(a.x) + (int64_t)b * a.sb + (int64_t)h * a.sh + (int64_t)cbi * a.cb * ss + 4 * lane;
    int pos = 0;
    bool bad = false;
    if (active) {

    // per-channel min / max over the block, two channels per instruction in the element type
    // (min/max of element-type values is exact, so the fp32 detour is not needed here)
    using T2 = typename QT<T>::T2;
    T2 lo01 = QT<T>::init2(INFINITY), lo23 = lo01, hi01 = QT<T>::init2(-INFINITY), hi23 = hi01;
#pragma unroll 8
    for (int t = 0; t < a.cb; t++) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(x + (int64_t)t * ss));
        const T2 v01 = *reinterpret_cast<const T2*>(&raw.x), v23 = *reinterpret_cast<const T2*>(&raw.y);
        lo01 = QT<T>::min2(lo01, v01); hi01 = QT<T>::max2(hi01, v01);
        lo23 = QT<T>::min2(lo23, v23); hi23 = QT<T>::max2(hi23, v23);
    }
    const float lo[4] = {QT<T>::lo_f(lo01), QT<T>::hi_f(lo01), QT<T>::lo_f(lo23), QT<T>::hi_f(lo23)};
    const float hi[4] = {QT<T>::lo_f(hi01), QT<T>::hi_f(hi01), QT<T>::lo_f(hi23), QT<T>::hi_f(hi23)};
    const Quantiser<T, HP> q0(lo[0], hi[0], a.rel), q1(lo[1], hi[1], a.rel), q2(lo[2], hi[2], a.rel), q3(lo[3], hi[3], a.rel);
    {
        const int64_t pi = (((int64_t)b * a.heads + h) * a.param_blocks + a.first_block + cbi) * 128 + 4 * lane;
        T sc[4] = {QT<T>::cvt(q0.scale), QT<T>::cvt(q1.scale), QT<T>::cvt(q2.scale), QT<T>::cvt(q3.scale)};
        T zr[4] = {QT<T>::cvt(q0.zero), QT<T>::cvt(q1.zero), QT<T>::cvt(q2.zero), QT<T>::cvt(q3.zero)};
        *reinterpret_cast<uint2*>(reinterpret_cast<T*>(a.scale) + pi) = *reinterpret_cast<const uint2*>(sc);
        *reinterpret_cast<uint2*>(reinterpret_cast<T*>(a.zero) + pi) = *reinterpret_cast<const uint2*>(zr);
    }
    bad = q0.degenerate() || q1.degenerate() || q2.degenerate() || q3.degenerate();
    const bool packable = __all_sync(0xffffffffu, q0.packable() && q1.packable() && q2.packable() && q3.packable());
    const bool half_ok = __all_sync(0xffffffffu, q0.half_domain() && q1.half_domain() && q2.half_domain() && q3.half_domain());
    // reordered blocks (order_block == cb here): the table of this block's rows
    const uint8_t* ordp = ORDERED ? a.order + ((int64_t)b * nctx + cbi) * a.cb : nullptr;
    if (!HP && half_ok) pos = k_encode_rounds_packed<T, BITS, true, ORDERED>(x, ss, ordp, q0, q1, q2, q3, g, stage, lane, bad);
    else if (!HP && packable) pos = k_encode_rounds_packed<T, BITS, false, ORDERED>(x, ss, ordp, q0, q1, q2, q3, g, stage, lane, bad);
    else pos = k_encode_rounds<T, HP, BITS, false, ORDERED>(x, ss, ordp, q0, q1, q2, q3, g, stage, lane, bad);
    __syncwarp();
    }   // active
    if (direct) {
        if (lane == 0) sh_sizes[wic] = (unsigned)pos;
        const int64_t left = per_seq - (int64_t)link * kKWarps;
        chain_store(a, b, link, sh_sizes, (int)(left < kKWarps ? left : kKWarps), &sh_word,
                    (int64_t)a.first_cb * a.heads + (int64_t)link * kKWarps, kKWarps, [&](int j) { return smem + j * slot_smem; });
    } else {
        store_slot(a.slots + (int64_t)warp * a.slot_stride, stage, pos, lane);
        if (lane == 0) a.info[((int64_t)b * a.info_seq_stride + (int64_t)(a.first_cb + cbi) * a.heads + h) * 2 + 1] = (unsigned)pos;
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(a.flags, kFlagCodeRange);
}

// ------------------------------------------------------------------------------------------ V
// one CTA per (sequence, token block): pass 1 computes the per-token parameters over all heads
// (one warp per token); pass 2 gives each warp whole V blocks (cb tokens x 64 channels): rows are
// quantised as they are loaded (8 channels of one token per lane, so the token's parameters are
// fetched once per 8 elements) into a uint8 tile in shared memory, from which the lane <-> channel
// packing reads its columns.
// Tile of one V block in shared memory, transposed for the packing stage: one row of CB bytes per
// channel, made of 16-byte chunks (one per pack); chunk p of channel ch is stored at chunk position
// p ^ v_swz(ch) so that both the word stores of the quantising stage and the 16-byte row reads of the
// packing stage spread over the banks.  Inside a chunk, byte 4*r0 + k holds token r0 + 4*k of the
// pack: the quantising lane with r0 = lane >> 3 owns those four tokens.
template <int CB>
__device__ __forceinline__ int v_swz(int ch) { return ((ch >> 1) ^ (ch >> 3)) & (CB / 16 - 1); }

// Quantises one V block into the tile.  Lane (r0 = lane >> 3, cg = lane & 7) loads 8 channels
// (16 bytes) of tokens r0, r0+4, r0+8, ... and, per pack, turns its 4 tokens x 8 channels into one
// 4-token word per channel.  PACKED: two channels per instruction (all tokens packable()).
// Returns the OR of all codes in 16-bit lanes for the range check.
template <typename T, int CB, int MODE>     // MODE 0: scalar conversion, 1: two elements per instruction in fp32, 2: in the element type
__device__ __forceinline__ unsigned v_quantise_tile(const T* src, int64_t ss, const float4* prm, const uint8_t* ord, uint8_t* tile, int lane) {
    constexpr bool PACKED = MODE == 1;
    const uint4* prmh = reinterpret_cast<const uint4*>(prm + CB);   // per token: r, -128*scale, r/128 (element-type pairs), code bias
    const int r0 = lane >> 3, cg = lane & 7;
    unsigned seen = 0;
    uint8_t* wr[4];                                        // row of channel 8cg + 2i at this lane's word, before the chunk swizzle
    int sw[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        wr[i] = tile + (8 * cg + 2 * i) * CB + 4 * r0;
        sw[i] = v_swz<CB>(8 * cg + 2 * i) << 4;           // channels 8cg + 2i and + 1 share the swizzle
    }
    const T* lsrc = src + 8 * cg;
#pragma unroll 1
    for (int p = 0; p < CB / 16; p++) {
        unsigned c[4][4];                                  // [token k][channel pair i] as 16-bit lanes
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int tok = 16 * p + 4 * k + r0;
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(lsrc + (int64_t)ord[tok] * ss));
            const unsigned rw[4] = {raw.x, raw.y, raw.z, raw.w};
            if (MODE == 2) {
                const uint4 ph = prmh[tok];
                HalfQuotient<T> hq;
                hq.r = *reinterpret_cast<const typename QT<T>::T2*>(&ph.x);
                hq.nsp = *reinterpret_cast<const typename QT<T>::T2*>(&ph.y);
                hq.rp = *reinterpret_cast<const typename QT<T>::T2*>(&ph.z);
                hq.kab = ph.w;
                hq.magic = QT<T>::dup((float)(QT<T>::kIntBits == 0x6600u ? 1536 : 192));
                hq.pre = QT<T>::dup(QT<T>::kPre);
#pragma unroll
                for (int i = 0; i < 4; i++) c[k][i] = hq.codes(rw[i]);
#pragma unroll
                for (int i = 0; i < 4; i++) seen |= c[k][i];
                continue;
            }
            const float4 pr = prm[tok];                    // scale, zero, 1/scale
            Quantiser<T, false> qz;
            qz.scale = pr.x; qz.zero = pr.y; qz.rcp = pr.z;
            if (PACKED) {
                const unsigned kab = __float_as_uint(pr.w);
#pragma unroll
                for (int i = 0; i < 4; i++) c[k][i] = packed_codes<T>(rw[i], qz, qz, kab);
            } else {
                const int zi = (int)pr.y;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = QT<T>::to_float2(rw[i]);
                    c[k][i] = qz.template code_u8<false>(f.x, zi) | (qz.template code_u8<false>(f.y, zi) << 16);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) seen |= c[k][i];
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // (even channel | odd channel) x tokens 0..3 -> one word per channel
            const unsigned x = __byte_perm(c[0][i], c[1][i], 0x6240), y = __byte_perm(c[2][i], c[3][i], 0x6240);
            uint8_t* at = wr[i] + ((p << 4) ^ sw[i]);
            *reinterpret_cast<unsigned*>(at) = __byte_perm(x, y, 0x5410);
            *reinterpret_cast<unsigned*>(at + CB) = __byte_perm(x, y, 0x7632);
        }
    }
    return seen;
}

// One 16-byte tile chunk (word r0: bytes k = codes of tokens r0 + 4k of the pack) -> the pack's
// minimum, bit length and 2*len-byte word (token 0 in the top bits).
template <int BITS>
__device__ __forceinline__ void chunk_to_pack(const uint4& cw, int& len, uint64_t& wd, unsigned& mn1) {
    const unsigned wv[4] = {cw.x, cw.y, cw.z, cw.w};
    unsigned mn = 0xFFFFFFFFu, mx = 0u;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const unsigned ev = wv[i] & 0x00FF00FFu, od = (wv[i] >> 8) & 0x00FF00FFu;
        mn = min_u16x2(mn, min_u16x2(ev, od));
        mx = max_u16x2(mx, max_u16x2(ev, od));
    }
    mn1 = min(mn & 0xFFFFu, mn >> 16);
    const unsigned mx1 = max(mx & 0xFFFFu, mx >> 16);
    len = min(bit_length_u32(mx1 - mn1), BITS);
    const unsigned step = 1u << len, rep = mn1 * 0x01010101u;
    // 16-bit slots: slot k collects tokens 4k..4k+3 (r0 = 0 highest) by Horner steps over the words
    unsigned zlo = 0, zhi = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const unsigned v = wv[i] - rep;
        zlo = zlo * step + __byte_perm(v, 0, 0x4140);
        zhi = zhi * step + __byte_perm(v, 0, 0x4342);
    }
    const unsigned wt = ((zlo & 0xFFFFu) << (4 * len)) | (zlo >> 16);     // tokens 0..7
    const unsigned wb = ((zhi & 0xFFFFu) << (4 * len)) | (zhi >> 16);     // tokens 8..15
    wd = ((uint64_t)wt << (8 * len)) | wb;
}

// Per-token quantisation parameters of one token block over all heads and channels (the
// reference's token mode reduces over dims [1, 4], utils/compute.py:405-410): half a warp per token.
// Writes (scale, zero, 1/scale, packed code bias or 0) to prm[] and scale / zero to the caller's arrays.
// ord[t] = source row (inside the block) of stored row t; WRITE = false keeps the parameters in shared memory only.
template <typename T, int CB, bool WRITE = true>
__device__ __forceinline__ bool token_params_pass(const FusedArgs& a, const T* xb, float4* prm, const uint8_t* ord, int b, int cbi, int lane, int wic) {
    bool bad = false;
    for (int t = 2 * wic + (lane >> 4); t < CB; t += 16) {     // 8 channels per lane
        const T* xt = xb + (int64_t)ord[t] * a.ss + 8 * (lane & 15);
        using T2 = typename QT<T>::T2;
        T2 lo2 = QT<T>::init2(INFINITY), hi2 = QT<T>::init2(-INFINITY);
#pragma unroll 4
        for (int h = 0; h < a.heads; h++) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xt + (int64_t)h * a.sh));
            const T2 v0 = *reinterpret_cast<const T2*>(&raw.x), v1 = *reinterpret_cast<const T2*>(&raw.y);
            const T2 v2 = *reinterpret_cast<const T2*>(&raw.z), v3 = *reinterpret_cast<const T2*>(&raw.w);
            lo2 = QT<T>::min2(lo2, QT<T>::min2(QT<T>::min2(v0, v1), QT<T>::min2(v2, v3)));
            hi2 = QT<T>::max2(hi2, QT<T>::max2(QT<T>::max2(v0, v1), QT<T>::max2(v2, v3)));
        }
        float lo = fminf(QT<T>::lo_f(lo2), QT<T>::hi_f(lo2)), hi = fmaxf(QT<T>::lo_f(hi2), QT<T>::hi_f(hi2));
#pragma unroll
        for (int s = 8; s > 0; s >>= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, s));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, s));
        }
        const Quantiser<T, false> qz(lo, hi, a.rel);
        bad = bad || qz.degenerate();
        if ((lane & 15) == 0) {
            prm[t] = make_float4(qz.scale, qz.zero, qz.rcp, __uint_as_float(qz.packable() ? packed_code_bias(qz, qz) : 0u));   // bias 0 = not packable
            const HalfQuotient<T> hq(qz, qz);
            reinterpret_cast<uint4*>(prm + CB)[t] = make_uint4(*reinterpret_cast<const unsigned*>(&hq.r), *reinterpret_cast<const unsigned*>(&hq.nsp),
                                                               *reinterpret_cast<const unsigned*>(&hq.rp), qz.half_domain() ? hq.kab : 0u);
            if (WRITE) {
                const int64_t pi = (int64_t)b * a.param_tokens + a.first_token + cbi * CB + t;
                reinterpret_cast<T*>(a.scale)[pi] = QT<T>::cvt(qz.scale);
                reinterpret_cast<T*>(a.zero)[pi] = QT<T>::cvt(qz.zero);
            }
        }
    }
    return bad;
}

// Source row (inside a block of CB tokens) of every stored row: the identity, or the caller's reorder of every
// order_block tokens.  256 threads; ends with a CTA barrier.
template <int CB>
__device__ __forceinline__ void load_row_order(const FusedArgs& a, uint8_t* ord, int b, int cbi) {
    for (int t = threadIdx.x; t < CB; t += 256) {
        unsigned src = t;
        if (a.order) {
            const int ob = a.order_block, sub = t / ob;
            src = sub * ob + a.order[((int64_t)b * (a.tokens / ob) + (int64_t)cbi * (CB / ob) + sub) * ob + (t - sub * ob)];
        }
        ord[t] = (uint8_t)src;
    }
    __syncthreads();
}

template <typename T, bool HP, int BITS, int CB>
__global__ void __launch_bounds__(256, 3) v_fused_encode_kernel(FusedArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int LB = len_field_bits(BITS);
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    const int nctx = a.tokens / CB;
    __shared__ unsigned sh_word, sh_sizes[16];
    const bool direct = a.status != nullptr;                 // then a warp keeps both of its blocks until the offsets are known
    int cbi = blockIdx.x, b = blockIdx.y;
    if (direct) chain_place(a, &sh_word, b, cbi);
    constexpr int PPT = CB == 32 ? 2 : 4, RPW = CB == 128 ? 2 : 1;
    const VGeom g(CB, BITS);
    const int bound16 = (g.head_bytes + g.nseg * (g.min_bytes + g.len_bytes + 32 * PPT * 2 * BITS) + 15) & ~15;
    const int wstride = CB * 64 + (direct ? 2 : 1) * bound16;
    float4* prm = reinterpret_cast<float4*>(smem);           // [cb] (scale, zero, 1/scale, fast)
    uint8_t* wbase = smem + 32 * CB + wic * wstride;
    uint8_t* ctile = wbase;                                  // [cb][64] codes
    const T* xb = reinterpret_cast<const T*>(a.x) + (int64_t)b * a.sb + (int64_t)cbi * CB * a.ss;
    uint8_t* ord = smem + 32 * CB + 8 * wstride;
    load_row_order<CB>(a, ord, b, cbi);

    // pass 1: per-token statistics across every head and channel
    bool bad = token_params_pass<T, CB>(a, xb, prm, ord, b, cbi, lane, wic);
    // one decision for the whole CTA: the packed conversion needs every token's parameters in range
    __syncthreads();
    bool mine_ok = true, mine_half = true;
    for (int t = threadIdx.x; t < CB; t += 256) {
        mine_ok = mine_ok && __float_as_uint(prm[t].w) != 0u;
        mine_half = mine_half && reinterpret_cast<const uint4*>(prm + CB)[t].w != 0u;
    }
    const bool all_packed = __syncthreads_and(mine_ok);
    const bool all_half = __syncthreads_and(mine_half);

    // pass 2: quantise + pack, one warp per V block
    unsigned seen = 0;
    const int nvb = 2 * a.heads;
    for (int vb = wic; vb < nvb; vb += 8) {
        const int h = vb >> 1, half = vb & 1;
        const T* src = xb + (int64_t)h * a.sh + 64 * half;
        uint8_t* stage = wbase + CB * 64 + (direct ? (vb >> 3) * bound16 : 0);
        __syncwarp();
        seen |= all_half ? v_quantise_tile<T, CB, 2>(src, a.ss, prm, ord, ctile, lane)
                         : all_packed ? v_quantise_tile<T, CB, 1>(src, a.ss, prm, ord, ctile, lane) : v_quantise_tile<T, CB, 0>(src, a.ss, prm, ord, ctile, lane);
        __syncwarp();
        int pos = g.head_bytes;
        unsigned seg_end = 0;
        for (int w = 0; w < 2; w++) {
            const int ch = 32 * w + lane;
            const uint8_t* row = ctile + ch * CB;
            const int swz = v_swz<CB>(ch);
            for (int r = 0; r < RPW; r++) {
                unsigned minword = 0, lenword = 0, lens4 = 0;
                uint64_t wd[4];
                int len[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    len[q] = 0; wd[q] = 0;
                    if (q < PPT) {
                        // word r0 of the chunk: bytes k = tokens r0 + 4k of the pack
                        const uint4 cw = *reinterpret_cast<const uint4*>(row + (((r * PPT + q) ^ swz) << 4));
                        unsigned mn1;
                        chunk_to_pack<BITS>(cw, len[q], wd[q], mn1);
                        minword |= (mn1 & ((1u << BITS) - 1u)) << (q * BITS);
                        lenword |= (unsigned)len[q] << (q * LB);
                        lens4 |= (unsigned)len[q] << (8 * q);
                    }
                }
                store_lane_fields_w<PPT * BITS>(stage + pos, lane, minword);
                store_lane_fields_w<PPT * LB>(stage + pos + g.min_bytes, lane, lenword);
                const unsigned inc = warp_inclusive_sum(lens4);
                const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
                const unsigned exc = inc - lens4;
                uint8_t* packs = stage + pos + g.min_bytes + g.len_bytes;
                unsigned before = 0;
#pragma unroll
                for (int q = 0; q < 4; q++)
                    if (q < PPT) {
                        store_pack_smem(packs + 2 * (before + ((exc >> (8 * q)) & 0xFFu)), wd[q], len[q]);
                        before += (tot >> (8 * q)) & 0xFFu;
                    }
                const unsigned seg_size = g.min_bytes + g.len_bytes + 2 * before;
                seg_end += seg_size;
                if (lane == 0) *reinterpret_cast<uint16_t*>(stage + 2 * (w * RPW + r)) = (uint16_t)seg_end;
                pos += seg_size;
            }
        }
        __syncwarp();
        if (direct) {
            if (lane == 0) sh_sizes[vb] = (unsigned)pos;
        } else {
            const int64_t blk = ((int64_t)b * nctx + cbi) * nvb + vb;
            store_slot(a.slots + blk * a.slot_stride, stage, pos, lane);
            if (lane == 0) a.info[((int64_t)b * a.info_seq_stride + (int64_t)(a.first_cb + cbi) * nvb + vb) * 2 + 1] = (unsigned)pos;
        }
    }
    if (direct)
        chain_store(a, b, cbi, sh_sizes, nvb, &sh_word, (int64_t)(a.first_cb + cbi) * nvb, 8,
                    [&](int j) { return smem + 32 * CB + (j & 7) * wstride + CB * 64 + (j >> 3) * bound16; });
    bad = bad || (seen & ~(((1u << BITS) - 1u) * 0x00010001u)) != 0;
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(a.flags, kFlagCodeRange);
}

// ------------------------------------------------------------------------- K, token mode
// K with per-token parameters (the reference's QuantMethod.PackKV pairing): the parameter pass and
// the quantising stage are V's; each warp then packs one K block (CB tokens x 128 channels of one
// head) in the K layout, lane = channels 4*lane..4*lane+3, one round per 16 tokens.
template <typename T, int BITS, int CB>
__global__ void __launch_bounds__(256, 2) kt_fused_encode_kernel(FusedArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int LB = len_field_bits(BITS);
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    const int nctx = a.tokens / CB;
    __shared__ unsigned sh_word, sh_sizes[8];
    const bool direct = a.status != nullptr;
    int cbi = blockIdx.x, b = blockIdx.y;
    if (direct) chain_place(a, &sh_word, b, cbi);
    const KGeom g(CB, BITS);
    const int bound16 = (g.head_bytes + g.rounds * (g.min_bytes + g.len_bytes + 128 * 2 * BITS) + 15) & ~15;
    float4* prm = reinterpret_cast<float4*>(smem);
    uint8_t* wbase = smem + 32 * CB + wic * (CB * 128 + bound16);
    uint8_t* ctile = wbase;                                  // two 64-channel halves of [64][CB] codes
    uint8_t* stage = wbase + CB * 128;
    const T* xb = reinterpret_cast<const T*>(a.x) + (int64_t)b * a.sb + (int64_t)cbi * CB * a.ss;
    uint8_t* ord = smem + 32 * CB + 8 * (CB * 128 + bound16);
    load_row_order<CB>(a, ord, b, cbi);

    bool bad = token_params_pass<T, CB>(a, xb, prm, ord, b, cbi, lane, wic);
    __syncthreads();
    bool mine_ok = true, mine_half = true;
    for (int t = threadIdx.x; t < CB; t += 256) {
        mine_ok = mine_ok && __float_as_uint(prm[t].w) != 0u;
        mine_half = mine_half && reinterpret_cast<const uint4*>(prm + CB)[t].w != 0u;
    }
    const bool all_packed = __syncthreads_and(mine_ok);
    const bool all_half = __syncthreads_and(mine_half);

    unsigned seen = 0;
    for (int h = wic; h < a.heads; h += 8) {
        const T* src = xb + (int64_t)h * a.sh;
        __syncwarp();
#pragma unroll 1
        for (int half = 0; half < 2; half++)
            seen |= all_half ? v_quantise_tile<T, CB, 2>(src + 64 * half, a.ss, prm, ord, ctile + half * 64 * CB, lane)
                             : all_packed ? v_quantise_tile<T, CB, 1>(src + 64 * half, a.ss, prm, ord, ctile + half * 64 * CB, lane)
                                          : v_quantise_tile<T, CB, 0>(src + 64 * half, a.ss, prm, ord, ctile + half * 64 * CB, lane);
        __syncwarp();
        // this lane's four channel rows and their chunk swizzles
        const uint8_t* row[4];
        int swz[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int ch = 4 * lane + j;
            row[j] = ctile + (ch >> 6) * 64 * CB + (ch & 63) * CB;
            swz[j] = v_swz<CB>(ch & 63);
        }
        int pos = g.head_bytes;
        unsigned round_end = 0;
        for (int r = 0; r < g.rounds; r++) {
            unsigned minword = 0, lenword = 0, lens4 = 0;
            uint64_t wd[4];
            int len[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint4 cw = *reinterpret_cast<const uint4*>(row[j] + ((r ^ swz[j]) << 4));
                unsigned mn1;
                chunk_to_pack<BITS>(cw, len[j], wd[j], mn1);
                minword |= (mn1 & ((1u << BITS) - 1u)) << (j * BITS);
                lenword |= (unsigned)len[j] << (j * LB);
                lens4 |= (unsigned)len[j] << (8 * j);
            }
            store_lane_fields_w<4 * BITS>(stage + pos, lane, minword);
            store_lane_fields_w<4 * LB>(stage + pos + g.min_bytes, lane, lenword);
            const unsigned inc = warp_inclusive_sum(lens4);
            const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
            const unsigned exc = inc - lens4;
            uint8_t* packs = stage + pos + g.min_bytes + g.len_bytes;
            unsigned before = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                store_pack_smem(packs + 2 * (before + ((exc >> (8 * j)) & 0xFFu)), wd[j], len[j]);
                before += (tot >> (8 * j)) & 0xFFu;
            }
            const unsigned round_size = g.min_bytes + g.len_bytes + 2 * before;
            round_end += round_size;
            if (lane == 0) *reinterpret_cast<uint16_t*>(stage + 2 * r) = (uint16_t)round_end;
            pos += round_size;
        }
        __syncwarp();
        if (direct) {
            if (lane == 0) sh_sizes[h] = (unsigned)pos;     // direct form: at most 8 heads, one block per warp
        } else {
            const int64_t blk = ((int64_t)b * nctx + cbi) * a.heads + h;
            store_slot(a.slots + blk * a.slot_stride, stage, pos, lane);
            if (lane == 0) a.info[((int64_t)b * a.info_seq_stride + (int64_t)(a.first_cb + cbi) * a.heads + h) * 2 + 1] = (unsigned)pos;
        }
    }
    if (direct)
        chain_store(a, b, cbi, sh_sizes, a.heads, &sh_word, (int64_t)(a.first_cb + cbi) * a.heads, 8,
                    [&](int j) { return smem + 32 * CB + j * (CB * 128 + bound16) + CB * 128; });
    bad = bad || (seen & ~(((1u << BITS) - 1u) * 0x00010001u)) != 0;
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(a.flags, kFlagCodeRange);
}

// ------------------------------------------------------------------------- order from values
// Token order of one block of 64 tokens by descending lower median of the V codes (stable on ties), the
// reference's median_repacking key (utils/compute.py:262-270), computed straight from fp16/bf16 V: per-token
// parameters as in the encoder, the token's heads*128 codes in registers (half a warp per token, 8 heads at
// most), then a binary search for the smallest m with count(code <= m) >= ceil(n / 2).  Same keys and the
// same order as median_order_kernel on the code matrix.  grid (tokens / 64, batch), 256 threads.
template <typename T>
__global__ void __launch_bounds__(256) value_median_order_kernel(FusedArgs a, uint8_t* order) {
    constexpr int CB = 64;
    __shared__ float4 prm[2 * CB];
    __shared__ uint8_t ident[CB];
    __shared__ uint8_t key[CB];
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    const int cbi = blockIdx.x, b = blockIdx.y;
    if (threadIdx.x < CB) ident[threadIdx.x] = (uint8_t)threadIdx.x;
    __syncthreads();
    const T* xb = reinterpret_cast<const T*>(a.x) + (int64_t)b * a.sb + (int64_t)cbi * CB * a.ss;
    token_params_pass<T, CB, false>(a, xb, prm, ident, b, cbi, lane, wic);
    __syncthreads();
    const int need = (a.heads * 128 + 1) / 2;
    const int n_slots = 16 * 64;                       // 16 lanes x 16 words x 4 codes per token; missing heads are filled with large codes
    const unsigned half_mask = 0xFFFFu << (lane & 16);
    for (int t = 2 * wic + (lane >> 4); t < CB; t += 16) {
        const float4 pr = prm[t];
        const uint4 ph = reinterpret_cast<const uint4*>(prm + CB)[t];
        const T* xt = xb + (int64_t)t * a.ss + 8 * (lane & 15);
        unsigned cw[16];
        // The token's codes, four per word.  Parameters inside the checked domain of the element-type quotient: two
        // codes per instruction, as in the encoder; otherwise (or if a code does not fit a byte) one by one in fp32.
        bool wide = ph.w == 0u, small = false;         // small: every code of this lane is known to be at most 15
        if (!wide) {
            HalfQuotient<T> hq;
            hq.r = *reinterpret_cast<const typename QT<T>::T2*>(&ph.x);
            hq.nsp = *reinterpret_cast<const typename QT<T>::T2*>(&ph.y);
            hq.rp = *reinterpret_cast<const typename QT<T>::T2*>(&ph.z);
            hq.kab = ph.w;
            hq.magic = QT<T>::dup((float)(QT<T>::kIntBits == 0x6600u ? 1536 : 192));
            hq.pre = QT<T>::dup(QT<T>::kPre);
            unsigned seen = 0;
#pragma unroll
            for (int h = 0; h < 8; h++) {
                cw[2 * h] = 0x7F7F7F7Fu; cw[2 * h + 1] = 0x7F7F7F7Fu;
                if (h < a.heads) {
                    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xt + (int64_t)h * a.sh));
                    const unsigned c0 = hq.codes(raw.x), c1 = hq.codes(raw.y), c2 = hq.codes(raw.z), c3 = hq.codes(raw.w);
                    seen |= c0 | c1 | c2 | c3;
                    cw[2 * h] = __byte_perm(c0, c1, 0x6420);
                    cw[2 * h + 1] = __byte_perm(c2, c3, 0x6420);
                }
            }
            wide = (seen & 0xFF80FF80u) != 0u;
            small = (seen & 0xFFF0FFF0u) == 0u;
        }
        if (__ballot_sync(0xffffffffu, wide) & half_mask) {          // the 16 lanes of a token decide together
            Quantiser<T, false> qz;
            qz.scale = pr.x; qz.zero = pr.y;
            qz.prepare();
            const int zi = (int)pr.y;
#pragma unroll
            for (int h = 0; h < 8; h++) {
                cw[2 * h] = 0x7F7F7F7Fu; cw[2 * h + 1] = 0x7F7F7F7Fu;       // heads that do not exist count as large codes
                if (h < a.heads) {
                    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(xt + (int64_t)h * a.sh));
                    const unsigned rw[4] = {raw.x, raw.y, raw.z, raw.w};
                    unsigned c[8];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f = QT<T>::to_float2(rw[i]);
                        c[2 * i] = min(qz.fast ? qz.template code_u8<true>(f.x, zi) : qz.template code_u8<false>(f.x, zi), 127u);
                        c[2 * i + 1] = min(qz.fast ? qz.template code_u8<true>(f.y, zi) : qz.template code_u8<false>(f.y, zi), 127u);
                    }
                    cw[2 * h] = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
                    cw[2 * h + 1] = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
                }
            }
        }
        // count(code <= m) over the token = slots - count(code > m); bit 7 of (code + 127 - m) is set iff code > m
        // (codes are at most 127); the flags of 16 words add up in four byte counters
        auto count_le = [&](int m) {
            const unsigned add = 0x01010101u * (unsigned)(127 - m);
            unsigned acc = 0;
#pragma unroll
            for (int i = 0; i < 16; i++) acc += ((cw[i] + add) >> 7) & 0x01010101u;
            unsigned over = (acc * 0x01010101u) >> 24;               // sum of the four byte counters (each at most 16)
#pragma unroll
            for (int s = 8; s > 0; s >>= 1) over += __shfl_xor_sync(0xffffffffu, over, s);
            return n_slots - (int)over;
        };
        int med = 16;                                  // codes above 15 are not expected (bits <= 4)
        // all of the token's codes at most 15: count_le(15) is the number of real codes, which is at least `need`
        // (decided for the warp's two tokens together: count_le shuffles over the whole warp)
        const bool all_small = __ballot_sync(0xffffffffu, !small) == 0u;
        const bool in_range = all_small || count_le(15) >= need;
        {
            // every lane runs every step (the counts shuffle over the whole warp, whose halves hold different tokens)
            int lo = 0, hi = 15;                       // smallest m in [lo, hi] with count_le(m) >= need
#pragma unroll
            for (int step = 0; step < 4; step++) {
                const int mid = (lo + hi) >> 1;
                if (count_le(mid) >= need) hi = mid; else lo = mid + 1;
            }
            if (in_range) med = hi;
        }
        if ((lane & 15) == 0) key[t] = (uint8_t)med;
    }
    __syncthreads();
    const int i = threadIdx.x;
    if (i < CB) {
        const int ki = key[i];
        int rank = 0;
        for (int j = 0; j < CB; j++) {
            const int kj = key[j];
            rank += (kj > ki) || (kj == ki && j < i);
        }
        order[((int64_t)b * (a.tokens / CB) + cbi) * CB + rank] = (uint8_t)i;
    }
}

// ------------------------------------------------------------------------------------ compact
// one warp per block: slot -> final offset in the sequence's stream
__global__ void __launch_bounds__(kWarpsPerCta * 32) compact_kernel(const uint8_t* slots, int slot_stride, uint8_t* stream,
                                                                    int64_t stream_seq_stride, int64_t capacity, const uint32_t* info,
                                                                    int64_t info_seq_stride, int first_blk, int blocks_per_seq, int batch,
                                                                    int slot_smem, unsigned* flags) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = lane_id(), wic = threadIdx.x >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + wic;
    if (warp >= (int64_t)blocks_per_seq * batch) return;
    const int b = (int)(warp / blocks_per_seq), i = (int)(warp % blocks_per_seq);
    const uint32_t* bi = info + ((int64_t)b * info_seq_stride + first_blk + i) * 2;
    const unsigned off = bi[0], size = bi[1];
    if ((int64_t)off + size > capacity) {
        if (lane == 0) atomicOr(flags, kFlagStreamOverflow);
        return;
    }
    uint8_t* dst = stream + (int64_t)b * stream_seq_stride + off;
    const uint8_t* src = slots + warp * slot_stride;          // 16-byte aligned
    // destination 16-byte chunks: chunk c covers block bytes [16c - phase, 16c - phase + 16)
    const int phase = (int)(reinterpret_cast<uintptr_t>(dst) & 15);   // even
    const int head = min((16 - phase) & 15, (int)size);               // bytes before the first aligned chunk
    for (int j = 2 * lane; j < head; j += 64) *reinterpret_cast<uint16_t*>(dst + j) = *reinterpret_cast<const uint16_t*>(src + j);
    const int nfull = ((int)size - head) >> 4;
    const unsigned* s32 = reinterpret_cast<const unsigned*>(src);
    const int sw = head >> 2;                                          // first source word of the body
    const unsigned sh = (unsigned)(head & 3) * 8;                      // 0 or 16: byte offset inside that word
    for (int c = lane; c < nfull; c += 32) {
        const unsigned* p = s32 + sw + 4 * c;                          // aligned 32-bit loads, realigned by funnel shifts
        const unsigned w0 = p[0], w1 = p[1], w2 = p[2], w3 = p[3], w4 = sh ? p[4] : 0u;   // the fifth word is past the slot when sh == 0
        *reinterpret_cast<uint4*>(dst + head + 16 * c) = make_uint4(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh),
                                                                    __funnelshift_r(w2, w3, sh), __funnelshift_r(w3, w4, sh));
    }
    for (int j = head + 16 * nfull + 2 * lane; j < (int)size; j += 64)
        *reinterpret_cast<uint16_t*>(dst + j) = *reinterpret_cast<const uint16_t*>(src + j);
}

// --------------------------------------------------------------------------------------- host
template <typename K>
static int opt_in_smem(K kernel, int bytes) {
    if (bytes > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return kCudaError;
    return kOk;
}

bool fused_encode_applicable(const FusedEncodeRequest& r) {
    if (r.high_precision_zero) return false;   // rare mode: served by the two-stage encoder
    if (r.bits < 2 || r.bits > 4) return false;
    if (r.cb != 32 && r.cb != 64 && r.cb != 128) return false;
    if (r.tokens % r.cb) return false;
    if (r.which == 0 && r.mode == 0 && r.qblock != r.cb) return false;       // K, channel mode: parameters per stream block
    if (r.which == 0 && r.mode != 0 && r.mode != 1) return false;
    if (r.which == 1 && r.mode != 1) return false;                           // V: per-token parameters
    if ((reinterpret_cast<uintptr_t>(r.x) & 15) || (r.stride_b & 7) || (r.stride_h & 7) || (r.stride_s & 7)) return false;
    return true;
}

int64_t fused_encode_scratch_bytes(const FusedEncodeRequest& r) {
    const int nblk = (r.tokens / r.cb) * r.heads * (r.which == 0 ? 1 : 2);
    const int bound = r.which == 0 ? KGeom(r.cb, r.bits).head_bytes + (r.cb / 16) * (16 * r.bits + 16 * len_field_bits(r.bits) + 256 * r.bits)
                                   : VGeom(r.cb, r.bits).head_bytes + VGeom(r.cb, r.bits).nseg * (VGeom(r.cb, r.bits).min_bytes + VGeom(r.cb, r.bits).len_bytes + 32 * VGeom(r.cb, r.bits).ppt * 2 * r.bits);
    return (int64_t)r.batch * nblk * ((bound + 15) & ~15);
}

template <typename T, bool HP, int BITS>
static int launch_fused_t(const FusedEncodeRequest& r, uint8_t* slots, const uint8_t* order, int order_block, cudaStream_t st) {
    FusedArgs a{};
    a.order = order; a.order_block = order_block;
    a.x = r.x; a.sb = r.stride_b; a.sh = r.stride_h; a.ss = r.stride_s;
    a.scale = r.scale; a.zero = r.zero;
    a.param_blocks = r.param_blocks; a.first_block = r.first_token / r.cb;
    a.param_tokens = r.param_tokens; a.first_token = r.first_token;
    a.slots = slots;
    a.info = r.block_info; a.info_seq_stride = r.info_seq_stride; a.first_cb = r.first_token / r.cb;
    a.batch = r.batch; a.heads = r.heads; a.tokens = r.tokens; a.cb = r.cb; a.bits = BITS; a.rel = r.rel; a.flags = r.flags;
    const int nctx = r.tokens / r.cb;
    int bound16, blocks_per_seq;
    // Direct form: the scratch holds only the ticket and the status array of the look-back.  The slots form stays
    // for more than 8 heads (a CTA of the per-token kernels would not hold all blocks of its token block), for
    // 128-token blocks in those kernels, for a scratch too small for the status array, and on request
    // (PKV_ENCODE_PATH=slots: measurements, tests).
    static const bool env_slots = [] { const char* v = std::getenv("PKV_ENCODE_PATH"); return v && std::string(v) == "slots"; }();
    const bool per_token_kernel = r.which == 1 || r.mode == 1;
    const int links = per_token_kernel ? nctx : (nctx * r.heads + kKWarps - 1) / kKWarps;
    const int64_t chain_bytes = 256 + (int64_t)r.batch * links * 8;
    // (128-token blocks in the per-token kernels: a second staging buffer per warp would leave one CTA per SM; measured
    // 2.55 ms against 2.28 ms for the slots form on the 4-bit sweep configuration)
    const bool direct = !env_slots && (!per_token_kernel || (r.heads <= 8 && r.cb != 128)) && chain_bytes <= fused_encode_scratch_bytes(r) &&
                        r.stream_bytes != nullptr;
    if (direct) {
        a.ticket = reinterpret_cast<unsigned*>(slots);
        a.status = reinterpret_cast<unsigned long long*>(slots + 256);
        a.links = links;
        a.stream = r.stream; a.stream_seq_stride = r.stream_seq_stride; a.capacity = r.capacity; a.stream_bytes = reinterpret_cast<unsigned*>(r.stream_bytes);
        if (cudaMemsetAsync(slots, 0, (size_t)chain_bytes, st) != cudaSuccess) return kCudaError;
    }
    if (r.which == 0) {
        const KGeom g(r.cb, BITS);
        bound16 = (g.head_bytes + g.rounds * (g.min_bytes + g.len_bytes + 128 * 2 * BITS) + 15) & ~15;
        a.slot_stride = bound16;
        blocks_per_seq = nctx * r.heads;
        const int64_t nwarps = (int64_t)blocks_per_seq * r.batch;
        const int smem = kKWarps * bound16 + 16;
        const unsigned grid = direct ? (unsigned)links * r.batch : (unsigned)((nwarps + kKWarps - 1) / kKWarps);
        if (r.mode == 1) {                       // per-token parameters: CTA per (sequence, token block)
            const int smem_t = 32 * r.cb + 8 * (r.cb * 128 + bound16) + r.cb + 16;
            auto launch_kt = [&](auto kern) {
                if (opt_in_smem(kern, smem_t)) return (int)kCudaError;
                kern<<<dim3(nctx, r.batch), 256, smem_t, st>>>(a);
                return (int)kOk;
            };
            int rc = kOk;
            if (r.cb == 32) rc = launch_kt(kt_fused_encode_kernel<T, BITS, 32>);
            else if (r.cb == 64) rc = launch_kt(kt_fused_encode_kernel<T, BITS, 64>);
            else rc = launch_kt(kt_fused_encode_kernel<T, BITS, 128>);
            if (rc != kOk) return rc;
        } else if (a.order) {
            auto kern = k_fused_encode_kernel<T, false, BITS, true>;
            if (opt_in_smem(kern, smem)) return kCudaError;
            kern<<<grid, kKWarps * 32, smem, st>>>(a);
        } else if (r.stride_s == 128) {
            auto kern = k_fused_encode_kernel<T, true, BITS>;
            if (opt_in_smem(kern, smem)) return kCudaError;
            kern<<<grid, kKWarps * 32, smem, st>>>(a);
        } else {
            auto kern = k_fused_encode_kernel<T, false, BITS>;
            if (opt_in_smem(kern, smem)) return kCudaError;
            kern<<<grid, kKWarps * 32, smem, st>>>(a);
        }
    } else {
        const VGeom g(r.cb, BITS);
        bound16 = (g.head_bytes + g.nseg * (g.min_bytes + g.len_bytes + 32 * g.ppt * 2 * BITS) + 15) & ~15;
        a.slot_stride = bound16;
        blocks_per_seq = nctx * 2 * r.heads;
        const int smem = 32 * r.cb + 8 * (r.cb * 64 + (direct ? 2 : 1) * bound16) + r.cb + 16;
        auto launch_v = [&](auto kern) {
            if (opt_in_smem(kern, smem)) return (int)kCudaError;
            kern<<<dim3(nctx, r.batch), 256, smem, st>>>(a);
            return (int)kOk;
        };
        int rc = kOk;
        if (r.cb == 32) rc = launch_v(v_fused_encode_kernel<T, HP, BITS, 32>);
        else if (r.cb == 64) rc = launch_v(v_fused_encode_kernel<T, HP, BITS, 64>);
        else rc = launch_v(v_fused_encode_kernel<T, HP, BITS, 128>);
        if (rc != kOk) return rc;
    }
    if (direct) return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
    // offsets: reuse the per-sequence scan of the two-pass encoder
    CodecShape sh{r.batch, r.tokens, r.heads * 128, r.cb, r.which == 0 ? 128 : 64, BITS, r.first_token / r.cb};
    CodecBuffers cbuf{nullptr, 0, r.stream, r.stream_seq_stride, r.capacity, r.block_info, r.info_seq_stride, r.stream_bytes, r.flags};
    int rc = launch_scan_sizes(sh, cbuf, st);
    if (rc != kOk) return rc;
    const int slot_smem = 0;
    const int64_t nwarps = (int64_t)blocks_per_seq * r.batch;
    const int per_cb = r.which == 0 ? r.heads : 2 * r.heads;
    compact_kernel<<<(unsigned)((nwarps + kWarpsPerCta - 1) / kWarpsPerCta), kWarpsPerCta * 32, 0, st>>>(
        slots, a.slot_stride, r.stream, r.stream_seq_stride, r.capacity, r.block_info, r.info_seq_stride, (r.first_token / r.cb) * per_cb,
        blocks_per_seq, r.batch, slot_smem, r.flags);
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

template <typename T, bool HP>
static int launch_fused_b(const FusedEncodeRequest& r, uint8_t* slots, const uint8_t* order, int order_block, cudaStream_t st) {
    switch (r.bits) {
        case 2: return launch_fused_t<T, HP, 2>(r, slots, order, order_block, st);
        case 3: return launch_fused_t<T, HP, 3>(r, slots, order, order_block, st);
        case 4: return launch_fused_t<T, HP, 4>(r, slots, order, order_block, st);
    }
    return kUnsupported;
}

int launch_fused_encode(const FusedEncodeRequest& r, uint8_t* slots, const uint8_t* order, int order_block, cudaStream_t st) {
    if (!fused_encode_applicable(r)) return kUnsupported;
    if (order) {
        // a reorder block must be a whole number of 16-token packs, fit a byte index, divide the stream block
        // and, for K with per-channel parameters, be the stream block itself
        if (order_block < 16 || order_block > 128 || order_block % 16 || r.cb % order_block || r.first_token % order_block) return kUnsupported;
        if (r.which == 0 && r.mode == 0 && order_block != r.cb) return kUnsupported;
        if (reinterpret_cast<uintptr_t>(order) & 15) return kBadArgument;
    }
    if ((int64_t)r.batch * r.tokens == 0) return kOk;
    if (!r.x || !r.scale || !r.zero || !r.stream || !r.block_info || !r.stream_bytes || !r.flags || !slots) return kBadArgument;
    if ((reinterpret_cast<uintptr_t>(slots) & 15) || (reinterpret_cast<uintptr_t>(r.stream) & 1) || (r.stream_seq_stride & 1)) return kBadArgument;
    return r.is_bf16 ? launch_fused_b<__nv_bfloat16, false>(r, slots, order, order_block, st) : launch_fused_b<__half, false>(r, slots, order, order_block, st);
}

#ifdef PKV_DEBUG_CHAIN
extern "C" int pkv_debug_chain_stats(unsigned long long* out4, int reset) {
    if (cudaMemcpyFromSymbol(out4, g_chain_stats, 32) != cudaSuccess) return -1;
    if (reset) { unsigned long long z[4] = {0, 0, 0, 0}; cudaMemcpyToSymbol(g_chain_stats, z, 32); }
    return 0;
}
#endif

int launch_value_median_order(const FusedEncodeRequest& r, uint8_t* order, int block, cudaStream_t st) {
    if (block != 64 || r.heads < 1 || r.heads > 8 || r.tokens % 64 || r.high_precision_zero) return kUnsupported;
    if (r.batch < 0 || r.tokens < 0) return kBadArgument;
    if ((int64_t)r.batch * r.tokens == 0) return kOk;
    if (!r.x || !order || (reinterpret_cast<uintptr_t>(r.x) & 15) || (r.stride_b & 7) || (r.stride_h & 7) || (r.stride_s & 7)) return kBadArgument;
    FusedArgs a{};
    a.x = r.x; a.sb = r.stride_b; a.sh = r.stride_h; a.ss = r.stride_s;
    a.batch = r.batch; a.heads = r.heads; a.tokens = r.tokens; a.cb = 64; a.rel = r.rel; a.flags = r.flags;
    if (r.is_bf16) value_median_order_kernel<__nv_bfloat16><<<dim3(r.tokens / 64, r.batch), 256, 0, st>>>(a, order);
    else value_median_order_kernel<__half><<<dim3(r.tokens / 64, r.batch), 256, 0, st>>>(a, order);
    return cudaGetLastError() == cudaSuccess ? kOk : kCudaError;
}

}  // namespace pkv
