/*
 * CPU oracle for the PackKV bit-pack codec.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C with run-time parameters, the byte format that the
 * reference's CPU codec writes and reads:
 *   packkv_cuda_ext/src/k_encode_cpu.cpp:11-231   (K encoder)
 *   packkv_cuda_ext/src/k_decode_cpu.cpp:11-225   (K decoder)
 *   packkv_cuda_ext/src/v_encode_cpu.cpp:11-259   (V encoder)
 *   packkv_cuda_ext/src/v_decode_cpu.cpp:11-216   (V decoder)
 *   packkv_cuda_ext/include/utils.h:24-36         (bits of the per-pack length field)
 *
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may call it; the
 * product never does.  Parity status: pinned.  For every configuration the reference's
 * templates instantiate (K: bits 2/3/4, token block 32/64/128; V: bits 2/3/4, token block
 * 128) the tests compare this restatement byte for byte with the reference's own sources
 * compiled into oracle/_ref, and with committed fixtures made from them.  The V formats
 * with a token block of 64 or 32 have no reference bitstream (the reference hard-codes two
 * 64-token half blocks per lane, v_encode_cpu.cpp:145); they are defined here by the same
 * rules and are "parity unpinned" against the reference.
 *
 * Format summary (all integers little-endian):
 *   pack  = 16 consecutive tokens of one channel.  min = smallest code, len =
 *           bit_length(max - min), word W = sum_i (code_i - min) << (len * (15 - i)),
 *           stored as 2*len bytes.
 *   field arrays: each of the 32 lanes owns `ppt` packs; its `ppt` fields of `fbits` bits
 *           (field i at bit i*fbits) form one lane word, and lane l's word sits at bit
 *           l*ppt*fbits of a little-endian bit string.
 *   K block (cb tokens x 128 channels), R = cb/16 rounds:
 *           u16 round_end[R] (cumulative round sizes), then per round: mins (fbits=bits),
 *           lens (fbits=bit_length(bits)), then packs ordered j=0..3, lane=0..31 for
 *           channel 4*lane+j.
 *   V block (cb tokens x 64 channels): lanes of warp w own channel 32*w+lane; a segment
 *           (w, r) covers `ppt` packs (ppt*16 tokens): u16 seg_end[2*rpw] cumulative in
 *           the order (w0,r0),(w0,r1),(w1,r0),(w1,r1); per segment mins, lens, then packs
 *           ordered p=0..ppt-1, lane=0..31.  cb=128: rpw=2, ppt=4 (the reference's only
 *           case); cb=64: rpw=1, ppt=4; cb=32: rpw=1, ppt=2.
 *   block_info[blk] = (byte offset, byte size), blk = ctx_block * (hidden/hb) + hidden_block;
 *           blocks are laid back to back with no padding.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>

#define PACK_TOKENS 16
#define LANES 32

static unsigned bit_length(unsigned v) {
    unsigned n = 0;
    while (v) { n++; v >>= 1; }
    return n;
}

/* utils.h:24-36 evaluates to bit_length(raw_bits) for raw_bits >= 1. */
static unsigned len_field_bits(unsigned raw_bits) {
    unsigned b = bit_length(raw_bits);
    return b ? b : 1;
}

static void put_bits(uint8_t *dst, size_t bitpos, unsigned nbits, unsigned value) {
    for (unsigned i = 0; i < nbits; i++) {
        size_t p = bitpos + i;
        if ((value >> i) & 1u) dst[p >> 3] |= (uint8_t)(1u << (p & 7));
    }
}

static unsigned get_bits(const uint8_t *src, size_t bitpos, unsigned nbits) {
    unsigned v = 0;
    for (unsigned i = 0; i < nbits; i++) {
        size_t p = bitpos + i;
        v |= (unsigned)((src[p >> 3] >> (p & 7)) & 1u) << i;
    }
    return v;
}

/* min and len of one pack; codes strided by `stride` bytes between tokens. */
static void pack_stats(const uint8_t *codes, size_t stride, unsigned *mn, unsigned *len) {
    unsigned lo = codes[0], hi = codes[0];
    for (int i = 1; i < PACK_TOKENS; i++) {
        unsigned c = codes[(size_t)i * stride];
        if (c < lo) lo = c;
        if (c > hi) hi = c;
    }
    *mn = lo;
    *len = bit_length(hi - lo);
}

static size_t put_pack(uint8_t *dst, const uint8_t *codes, size_t stride, unsigned mn, unsigned len) {
    uint64_t w = 0;
    for (int i = 0; i < PACK_TOKENS; i++) {
        w <<= len;
        w |= (uint64_t)(codes[(size_t)i * stride] - mn);
    }
    size_t nbytes = 2u * len;
    for (size_t b = 0; b < nbytes; b++) { dst[b] = (uint8_t)(w & 0xFF); w >>= 8; }
    return nbytes;
}

static size_t get_pack(const uint8_t *src, uint8_t *codes, size_t stride, unsigned mn, unsigned len) {
    uint64_t w = 0;
    size_t nbytes = 2u * len;
    for (size_t b = 0; b < nbytes; b++) w |= (uint64_t)src[b] << (8 * b);
    uint64_t mask = (len >= 64) ? ~0ull : ((1ull << len) - 1);
    for (int i = PACK_TOKENS - 1; i >= 0; i--) {
        codes[(size_t)i * stride] = (uint8_t)((w & mask) + mn);
        w >>= len;
    }
    return nbytes;
}

static int k_args_ok(int64_t ctx_len, int64_t hidden, int cb, int hb, int bits) {
    if (hb != 128) return 0;
    if (cb <= 0 || cb % PACK_TOKENS) return 0;
    if (bits < 2 || bits > 4) return 0;
    if (ctx_len < 0 || hidden <= 0 || ctx_len % cb || hidden % hb) return 0;
    return 1;
}

static int v_geometry(int cb, int *rpw, int *ppt) {
    if (cb == 128) { *rpw = 2; *ppt = 4; return 1; }
    if (cb == 64)  { *rpw = 1; *ppt = 4; return 1; }
    if (cb == 32)  { *rpw = 1; *ppt = 2; return 1; }
    return 0;
}

static int v_args_ok(int64_t ctx_len, int64_t hidden, int cb, int hb, int bits) {
    int rpw, ppt;
    if (hb != 64) return 0;
    if (!v_geometry(cb, &rpw, &ppt)) return 0;
    if (bits < 2 || bits > 4) return 0;
    if (ctx_len < 0 || hidden <= 0 || ctx_len % cb || hidden % hb) return 0;
    return 1;
}

/* One K block.  `blk` points at code (token 0, channel 0) of the block. */
static size_t k_block_encode(const uint8_t *blk, size_t row_stride, int cb, int bits, uint8_t *out) {
    const int rounds = cb / PACK_TOKENS;
    const unsigned lbits = len_field_bits((unsigned)bits);
    const size_t min_bytes = (size_t)bits * 128 / 8, len_bytes = (size_t)lbits * 128 / 8;
    size_t off = 2u * (size_t)rounds;
    uint16_t round_end = 0;
    for (int r = 0; r < rounds; r++) {
        unsigned mn[128], ln[128];
        const uint8_t *rows = blk + (size_t)r * PACK_TOKENS * row_stride;
        for (int c = 0; c < 128; c++) pack_stats(rows + c, row_stride, &mn[c], &ln[c]);
        uint8_t *mins = out + off, *lens = mins + min_bytes, *packs = lens + len_bytes;
        memset(mins, 0, min_bytes + len_bytes);
        for (int lane = 0; lane < LANES; lane++)
            for (int i = 0; i < 4; i++) {
                put_bits(mins, (size_t)(lane * 4 + i) * bits, (unsigned)bits, mn[lane * 4 + i]);
                put_bits(lens, (size_t)(lane * 4 + i) * lbits, lbits, ln[lane * 4 + i]);
            }
        size_t p = 0;
        for (int j = 0; j < 4; j++)
            for (int lane = 0; lane < LANES; lane++) {
                int c = lane * 4 + j;
                p += put_pack(packs + p, rows + c, row_stride, mn[c], ln[c]);
            }
        size_t round_size = min_bytes + len_bytes + p;
        off += round_size;
        round_end = (uint16_t)(round_end + round_size);
        out[2 * r] = (uint8_t)(round_end & 0xFF);
        out[2 * r + 1] = (uint8_t)(round_end >> 8);
    }
    return off;
}

static void k_block_decode(const uint8_t *in, uint8_t *blk, size_t row_stride, int cb, int bits) {
    const int rounds = cb / PACK_TOKENS;
    const unsigned lbits = len_field_bits((unsigned)bits);
    const size_t min_bytes = (size_t)bits * 128 / 8, len_bytes = (size_t)lbits * 128 / 8;
    size_t off = 2u * (size_t)rounds;
    for (int r = 0; r < rounds; r++) {
        const uint8_t *mins = in + off, *lens = mins + min_bytes, *packs = lens + len_bytes;
        uint8_t *rows = blk + (size_t)r * PACK_TOKENS * row_stride;
        size_t p = 0;
        for (int j = 0; j < 4; j++)
            for (int lane = 0; lane < LANES; lane++) {
                int c = lane * 4 + j;
                unsigned mn = get_bits(mins, (size_t)c * bits, (unsigned)bits);
                unsigned ln = get_bits(lens, (size_t)c * lbits, lbits);
                p += get_pack(packs + p, rows + c, row_stride, mn, ln);
            }
        off += min_bytes + len_bytes + p;
    }
}

static size_t v_block_encode(const uint8_t *blk, size_t row_stride, int cb, int bits, uint8_t *out) {
    int rpw = 1, ppt = 4;
    v_geometry(cb, &rpw, &ppt);
    const unsigned lbits = len_field_bits((unsigned)bits);
    const size_t min_bytes = (size_t)bits * ppt * LANES / 8, len_bytes = (size_t)lbits * ppt * LANES / 8;
    const int nseg = 2 * rpw;
    size_t off = 2u * (size_t)nseg;
    uint16_t seg_end = 0;
    for (int w = 0; w < 2; w++)
        for (int r = 0; r < rpw; r++) {
            unsigned mn[LANES][4], ln[LANES][4];
            for (int lane = 0; lane < LANES; lane++)
                for (int p = 0; p < ppt; p++) {
                    const uint8_t *src = blk + (size_t)(r * ppt + p) * PACK_TOKENS * row_stride + (w * LANES + lane);
                    pack_stats(src, row_stride, &mn[lane][p], &ln[lane][p]);
                }
            uint8_t *mins = out + off, *lens = mins + min_bytes, *packs = lens + len_bytes;
            memset(mins, 0, min_bytes + len_bytes);
            for (int lane = 0; lane < LANES; lane++)
                for (int p = 0; p < ppt; p++) {
                    put_bits(mins, (size_t)(lane * ppt + p) * bits, (unsigned)bits, mn[lane][p]);
                    put_bits(lens, (size_t)(lane * ppt + p) * lbits, lbits, ln[lane][p]);
                }
            size_t q = 0;
            for (int p = 0; p < ppt; p++)
                for (int lane = 0; lane < LANES; lane++) {
                    const uint8_t *src = blk + (size_t)(r * ppt + p) * PACK_TOKENS * row_stride + (w * LANES + lane);
                    q += put_pack(packs + q, src, row_stride, mn[lane][p], ln[lane][p]);
                }
            size_t seg_size = min_bytes + len_bytes + q;
            off += seg_size;
            seg_end = (uint16_t)(seg_end + seg_size);
            int s = w * rpw + r;
            out[2 * s] = (uint8_t)(seg_end & 0xFF);
            out[2 * s + 1] = (uint8_t)(seg_end >> 8);
        }
    return off;
}

static void v_block_decode(const uint8_t *in, uint8_t *blk, size_t row_stride, int cb, int bits) {
    int rpw = 1, ppt = 4;
    v_geometry(cb, &rpw, &ppt);
    const unsigned lbits = len_field_bits((unsigned)bits);
    const size_t min_bytes = (size_t)bits * ppt * LANES / 8, len_bytes = (size_t)lbits * ppt * LANES / 8;
    size_t off = 2u * (size_t)(2 * rpw);
    for (int w = 0; w < 2; w++)
        for (int r = 0; r < rpw; r++) {
            const uint8_t *mins = in + off, *lens = mins + min_bytes, *packs = lens + len_bytes;
            size_t q = 0;
            for (int p = 0; p < ppt; p++)
                for (int lane = 0; lane < LANES; lane++) {
                    unsigned mn = get_bits(mins, (size_t)(lane * ppt + p) * bits, (unsigned)bits);
                    unsigned ln = get_bits(lens, (size_t)(lane * ppt + p) * lbits, lbits);
                    uint8_t *dst = blk + (size_t)(r * ppt + p) * PACK_TOKENS * row_stride + (w * LANES + lane);
                    q += get_pack(packs + q, dst, row_stride, mn, ln);
                }
            off += min_bytes + len_bytes + q;
        }
}

/* Worst-case bytes of one block; callers size buffers with it. */
int64_t pkv_oracle_k_block_bound(int cb, int bits) {
    const int rounds = cb / PACK_TOKENS;
    const unsigned lbits = len_field_bits((unsigned)bits);
    return 2 * rounds + (int64_t)rounds * ((int64_t)bits * 16 + lbits * 16 + 128 * 2 * bits);
}

int64_t pkv_oracle_v_block_bound(int cb, int bits) {
    int rpw, ppt;
    if (!v_geometry(cb, &rpw, &ppt)) return -1;
    const unsigned lbits = len_field_bits((unsigned)bits);
    const int nseg = 2 * rpw;
    return 2 * nseg + (int64_t)nseg * ((int64_t)bits * ppt * 4 + lbits * ppt * 4 + LANES * ppt * 2 * bits);
}

/* codes: (ctx_len, hidden) row-major u8.  Returns total bytes, or -1 for a bad argument. */
int64_t pkv_oracle_k_encode(const uint8_t *codes, uint8_t *out, uint32_t *info,
                            int64_t ctx_len, int64_t hidden, int cb, int hb, int bits) {
    if (!k_args_ok(ctx_len, hidden, cb, hb, bits)) return -1;
    const int64_t nctx = ctx_len / cb, nhid = hidden / hb;
    size_t total = 0;
    for (int64_t cbi = 0; cbi < nctx; cbi++)
        for (int64_t hbi = 0; hbi < nhid; hbi++) {
            const uint8_t *blk = codes + (size_t)cbi * cb * hidden + (size_t)hbi * hb;
            size_t sz = k_block_encode(blk, (size_t)hidden, cb, bits, out + total);
            info[2 * (cbi * nhid + hbi)] = (uint32_t)total;
            info[2 * (cbi * nhid + hbi) + 1] = (uint32_t)sz;
            total += sz;
        }
    return (int64_t)total;
}

int pkv_oracle_k_decode(const uint8_t *in, const uint32_t *info, uint8_t *codes,
                        int64_t ctx_len, int64_t hidden, int cb, int hb, int bits) {
    if (!k_args_ok(ctx_len, hidden, cb, hb, bits)) return -1;
    const int64_t nctx = ctx_len / cb, nhid = hidden / hb;
    for (int64_t cbi = 0; cbi < nctx; cbi++)
        for (int64_t hbi = 0; hbi < nhid; hbi++) {
            uint8_t *blk = codes + (size_t)cbi * cb * hidden + (size_t)hbi * hb;
            k_block_decode(in + info[2 * (cbi * nhid + hbi)], blk, (size_t)hidden, cb, bits);
        }
    return 0;
}

int64_t pkv_oracle_v_encode(const uint8_t *codes, uint8_t *out, uint32_t *info,
                            int64_t ctx_len, int64_t hidden, int cb, int hb, int bits) {
    if (!v_args_ok(ctx_len, hidden, cb, hb, bits)) return -1;
    const int64_t nctx = ctx_len / cb, nhid = hidden / hb;
    size_t total = 0;
    for (int64_t cbi = 0; cbi < nctx; cbi++)
        for (int64_t hbi = 0; hbi < nhid; hbi++) {
            const uint8_t *blk = codes + (size_t)cbi * cb * hidden + (size_t)hbi * hb;
            size_t sz = v_block_encode(blk, (size_t)hidden, cb, bits, out + total);
            info[2 * (cbi * nhid + hbi)] = (uint32_t)total;
            info[2 * (cbi * nhid + hbi) + 1] = (uint32_t)sz;
            total += sz;
        }
    return (int64_t)total;
}

int pkv_oracle_v_decode(const uint8_t *in, const uint32_t *info, uint8_t *codes,
                        int64_t ctx_len, int64_t hidden, int cb, int hb, int bits) {
    if (!v_args_ok(ctx_len, hidden, cb, hb, bits)) return -1;
    const int64_t nctx = ctx_len / cb, nhid = hidden / hb;
    for (int64_t cbi = 0; cbi < nctx; cbi++)
        for (int64_t hbi = 0; hbi < nhid; hbi++) {
            uint8_t *blk = codes + (size_t)cbi * cb * hidden + (size_t)hbi * hb;
            v_block_decode(in + info[2 * (cbi * nhid + hbi)], blk, (size_t)hidden, cb, bits);
        }
    return 0;
}
