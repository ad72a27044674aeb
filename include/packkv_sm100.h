/*
 * C ABI of libpackkv_sm100.so -- the B200 (sm_100a) implementation of PackKV's compression
 * hot path.  Plain pointers and sizes only; every pointer is a DEVICE pointer unless the
 * parameter name ends in _host.  Every call is asynchronous on `cuda_stream` (a
 * cudaStream_t passed as void*; NULL = the legacy default stream) and allocates nothing.
 *
 * Return value: PKV_OK, or a PKV_ERR_* code for arguments that can be rejected on the host.
 * Conditions only the kernels can see (a block that does not fit the stream, a code that
 * does not fit `bits`, a corrupt block_info entry) are OR-ed as PKV_FLAG_* bits into the
 * caller's device word `dev_flags`, and the offending block is skipped; nothing aborts.
 *
 * Each declaration cites the reference interface it replaces (paths inside the PackKV
 * repository).
 */
#ifndef PACKKV_SM100_H
#define PACKKV_SM100_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PKV_OK 0
#define PKV_ERR_BAD_ARGUMENT 1
#define PKV_ERR_UNSUPPORTED 2   /* the reference raises RuntimeError("not supported") here */
#define PKV_ERR_CUDA 3
#define PKV_ERR_TOO_LARGE 4     /* pkv_encode_tensor_static: the call needs more than the built-in scratch */

#define PKV_FLAG_STREAM_OVERFLOW 1u
#define PKV_FLAG_CODE_RANGE 2u
#define PKV_FLAG_BAD_STREAM 4u
#define PKV_FLAG_TIMEOUT 8u
#define PKV_FLAG_ZERO_RANGE 16u   /* pkv_decode_attention: a zero-point too large for the exact in-kernel dequantisation */

/* quantisation modes (the reference's QuantMode, utils/compute.py:6-11).  ChannelQuant and TokenQuant are the modes of
 * its two quantisation methods and the only ones the single-pass encoder and the attention kernel take; VectorQuant
 * and BlockQuant are served by pkv_quantize / pkv_dequantize (and the codec entry points on the code matrix). */
#define PKV_K_CHANNEL 0
#define PKV_K_TOKEN 1
#define PKV_Q_VECTOR 2
#define PKV_Q_BLOCK 3

/* Library / build identification: returns the ABI version (currently 1). */
int32_t pkv_abi_version(void);

/*
 * Bit-pack encoders.  Replace k_encode_cpu_pyi (packkv_cuda_ext/src/k_encode_cpu.cpp:286-331)
 * and v_encode_cpu_pyi (packkv_cuda_ext/src/v_encode_cpu.cpp:301-346); the byte stream and
 * block_info are identical to theirs.
 *
 * `n_seq` independent sequences are encoded in one call.  Sequence s reads the uint8 code
 * matrix (ctx_len, hidden) at codes + s*codes_seq_stride, appends its blocks to the stream at
 * stream + s*stream_seq_stride (at most `capacity` bytes), and fills block_info rows
 * [first_cb*(hidden/hb), ...) of its table at block_info + 2*s*info_seq_stride.
 * stream_bytes[s] is the running stream length: read when first_cb > 0 (append), written
 * always.  Block shapes: K hb=128, cb in {32,64,128}; V hb=64, cb in {32,64,128}; bits 2..4.
 * codes must be 16-byte aligned, streams 2-byte aligned.
 */
int32_t pkv_k_encode(const uint8_t* codes, int64_t codes_seq_stride, uint8_t* stream, int64_t stream_seq_stride,
                     int64_t capacity, uint32_t* block_info, int64_t info_seq_stride, uint32_t* stream_bytes,
                     uint32_t* dev_flags, int32_t n_seq, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb,
                     int32_t bits, int32_t first_cb, void* cuda_stream);
int32_t pkv_v_encode(const uint8_t* codes, int64_t codes_seq_stride, uint8_t* stream, int64_t stream_seq_stride,
                     int64_t capacity, uint32_t* block_info, int64_t info_seq_stride, uint32_t* stream_bytes,
                     uint32_t* dev_flags, int32_t n_seq, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb,
                     int32_t bits, int32_t first_cb, void* cuda_stream);

/*
 * Bit-pack decoders.  Replace k_decode_cpu_pyi (packkv_cuda_ext/src/k_decode_cpu.cpp:281-326)
 * and v_decode_cpu_pyi (packkv_cuda_ext/src/v_decode_cpu.cpp:258-303).  `capacity` is the
 * number of valid stream bytes per sequence; entries pointing outside it are skipped and
 * flagged.
 */
int32_t pkv_k_decode(const uint8_t* stream, int64_t stream_seq_stride, int64_t capacity, const uint32_t* block_info,
                     int64_t info_seq_stride, uint8_t* codes, int64_t codes_seq_stride, uint32_t* dev_flags,
                     int32_t n_seq, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb, int32_t bits,
                     int32_t first_cb, void* cuda_stream);
int32_t pkv_v_decode(const uint8_t* stream, int64_t stream_seq_stride, int64_t capacity, const uint32_t* block_info,
                     int64_t info_seq_stride, uint8_t* codes, int64_t codes_seq_stride, uint32_t* dev_flags,
                     int32_t n_seq, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb, int32_t bits,
                     int32_t first_cb, void* cuda_stream);

/*
 * The reference's two-step GPU API, kept for its callers (evaluation/evaluation.py:398-715).
 * pkv_kq_mat_vec_mul replaces kq_mat_vec_mul (packkv_cuda_ext/src/kernels.cu:611-630):
 *   kq_out[h, n] = sum_d q[h, d] * code[n, h*128 + d], q given in the reference's lane-permuted
 *   order (evaluation.py:465-468), kq_out (hidden/128, ctx_len) in the element type.
 * pkv_wv_mat_vec_mul replaces wv_mat_vec_mul (kernels.cu:842-859):
 *   wv_out[c] += sum_n w[c/128, n] * code[n, c], wv_out (hidden) float32, accumulated into.
 * One sequence per call; `stream_bytes` = valid bytes of the stream (16-byte aligned base).
 * Unlike the reference these do not synchronise or time themselves.
 */
int32_t pkv_kq_mat_vec_mul(const uint8_t* stream, int64_t stream_bytes, const uint32_t* block_info, const void* q,
                           void* kq_out, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb, int32_t bits,
                           int32_t is_bf16, uint32_t* dev_flags, void* cuda_stream);
int32_t pkv_wv_mat_vec_mul(const uint8_t* stream, int64_t stream_bytes, const uint32_t* block_info, const void* w,
                           float* wv_out, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb, int32_t bits,
                           int32_t is_bf16, uint32_t* dev_flags, void* cuda_stream);
/*
 * pkv_fused_kq replaces fused_kq_launcher (packkv_cuda_ext/src/fused_kernels.cu:171-185):
 *   our_kq[m, n] = (sum_d q[m, d] * zero[n] + t[m, n]) * scale[n];  q (M, K), t and our_kq (M, N).
 * pkv_fused_wv replaces fused_wv_launcher (fused_kernels.cu:355-369):
 *   our_wv[m, d] = sum_n w[m, n] * zero[n] * scale[n] + term1[m, d];  w (M, N), term1 and our_wv (M, D).
 * Any M, N, K, D (the reference accepts only M in {8, 40} and K = D = 128).
 */
int32_t pkv_fused_kq(void* our_kq, const void* q, const void* zero, const void* scale, const void* t, int32_t M,
                     int32_t N, int32_t K, int32_t is_bf16, void* cuda_stream);
int32_t pkv_fused_wv(void* our_wv, const void* w, const void* zero, const void* scale, const void* term1, int32_t M,
                     int32_t N, int32_t D, int32_t is_bf16, void* cuda_stream);

/*
 * Block quantiser: fp16/bf16 K or V (batch, heads, tokens, 128) -> uint8 codes laid out as the
 * encoders' input (batch, tokens, heads*128), plus scale and zero-point in the element type.
 * Replaces quant_ints (utils/compute.py:84-112) bit for bit, including the rounding to the
 * element type after every op.  mode PKV_K_CHANNEL: parameters per (sequence, head, token
 * block, channel), written to (batch, heads, param_blocks, 128) starting at block first_block;
 * mode PKV_K_TOKEN: per (sequence, token) across all heads, written to (batch, param_tokens)
 * starting at token first_token; mode PKV_Q_VECTOR: per (sequence, head, token) across its 128 channels, written to
 * (batch, heads, param_tokens) starting at token first_token; mode PKV_Q_BLOCK: per (sequence, token block) across
 * heads and channels, written to (batch, param_blocks) starting at block first_block (the reduction sets of
 * QUANT_DIM, utils/compute.py:405-410).  x strides are in elements; rows of 128 channels are
 * contiguous and 8-byte aligned.  bits > 0 enables the range check (PKV_FLAG_CODE_RANGE).
 */
int32_t pkv_quantize(const void* x, int64_t stride_b, int64_t stride_h, int64_t stride_s, uint8_t* codes,
                     int64_t codes_seq_stride, void* scale, void* zero, int32_t param_blocks, int32_t first_block,
                     int32_t param_tokens, int32_t first_token, int32_t batch, int32_t heads, int32_t tokens,
                     int32_t block, float rel, int32_t bits, int32_t mode, int32_t high_precision_zero,
                     int32_t is_bf16, uint32_t* dev_flags, void* cuda_stream);

/*
 * In-block token reordering; replaces median_repacking (utils/compute.py:262-270).
 * pkv_median_order: key[token] = lower median of the token's V codes (all heads, all channels),
 *   order[b][block][rank] = index inside the block of the token with that rank when sorted by key,
 *   descending, ties in original order (torch's unstable sort leaves tie order unspecified).
 *   v_codes (batch, tokens, heads*128) uint8 with codes <= 15; block <= 128; keys may be NULL.
 * pkv_gather_rows: dst row (block*B + r) <- src row (block*B + order[r]) for code matrices
 *   (row_bytes = heads*128); pkv_gather_params: the same gather for per-token fp16/bf16 parameter
 *   arrays (batch, row_len), applied to tokens [first, first+tokens).  src and dst must differ.
 */
int32_t pkv_median_order(const uint8_t* v_codes, int64_t codes_seq_stride, uint8_t* order, uint8_t* keys,
                         int32_t batch, int32_t heads, int32_t tokens, int32_t block, void* cuda_stream);
int32_t pkv_gather_rows(const uint8_t* src, uint8_t* dst, int64_t seq_stride, const uint8_t* order, int32_t batch,
                        int32_t tokens, int32_t block, int32_t row_bytes, void* cuda_stream);
int32_t pkv_gather_params(const void* src, void* dst, int64_t row_len, int32_t first, const uint8_t* order,
                          int32_t batch, int32_t tokens, int32_t block, void* cuda_stream);

/*
 * Decode-step append to the uncompressed residual: rows [position, position + tokens) of k_res / v_res
 * (batch, heads, res_capacity, 128) receive the new K tokens after rotary embedding (the reference's
 * apply_rotary_pos_emb_single inside PackKVCachePytorchQuant.update, models/cache/packkv_quant.py:57-60;
 * cos = sin = NULL when the caller has rotated K already) and the new V tokens
 * (torch.cat of the buffers, utils/compute.py:160-163).  Strides in elements.
 */
int32_t pkv_append_residual(const void* k, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s, const void* v,
                            int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_s, const void* cos, const void* sin,
                            int64_t cs_stride_b, void* k_res, void* v_res, int64_t res_stride_b, int64_t res_stride_h,
                            int32_t res_capacity, int32_t position, int32_t batch, int32_t heads, int32_t tokens,
                            int32_t is_bf16, void* cuda_stream);

/*
 * pkv_greedy_order: the reference's greedy_repacking (utils/compute.py:210-260) per sequence and token
 *   block.  A token's feature vector is its K codes followed by its V codes (k_codes, v_codes:
 *   (batch, tokens, heads*128) uint8, same stride).  For every pack of pack_len tokens the seed is the
 *   remaining token with the largest cosine to the rounded mean of the remaining tokens; the others
 *   are picked one by one as the token that adds the fewest bits (sum over features of
 *   bit_length(max - min) of the pack); ties take the first remaining token.  order (batch,
 *   tokens/block, block) lists original in-block positions in picked order, usable with
 *   pkv_gather_rows / pkv_gather_params.  Comparisons are exact (integer / rational); the reference
 *   evaluates them in fp32, so the two can differ only where two cosines tie within fp32 rounding.
 * pkv_size_model: the reference's bit_pack size estimate (utils/compute.py:272-297) for one code
 *   tensor (batch, tokens, hidden) uint8: *bits_sum += sum over packs (pack_len consecutive tokens of
 *   one feature) of bit_length(max - min); present[8] |= bitmap of the code values that occur.  Both
 *   outputs are device memory the caller zeroes.  bytes = (bits_sum * pack_len + n_packs *
 *   (b + ceil(log2(b + 1)))) / 8 with b = ceil(log2(popcount(present))).
 */
int32_t pkv_greedy_order(const uint8_t* k_codes, const uint8_t* v_codes, int64_t codes_seq_stride, uint8_t* order,
                         int32_t batch, int32_t heads, int32_t tokens, int32_t block, int32_t pack_len, void* cuda_stream);
int32_t pkv_size_model(const uint8_t* codes, int64_t codes_seq_stride, int32_t batch, int32_t tokens, int32_t hidden,
                       int32_t pack_len, uint64_t* bits_sum, uint32_t* present, void* cuda_stream);

/*
 * One-call encoder: quantise x (batch, heads, tokens, 128) and bit-pack it behind the blocks
 * already in the streams.  Equivalent to pkv_quantize followed by pkv_k_encode (which = 0, blocks of
 * cb tokens x 128 channels) or pkv_v_encode (which = 1, cb x 64); replaces the reference's
 * quant_ints on the GPU + copy to the host + k/v_encode_cpu + copy back
 * (evaluation/evaluation.py:402-428, 591-618).  `codes_scratch` is caller-provided device scratch
 * of at least batch*tokens*heads*128 bytes (16-byte aligned) that holds the uint8 codes between the
 * two stages; its contents are unspecified afterwards.  first_token = tokens already encoded per
 * sequence (a multiple of cb and of qblock).
 */
typedef struct pkv_encode_args {
    const void* x; int64_t stride_b, stride_h, stride_s;     /* strides in elements */
    void* scale; void* zero; int32_t param_blocks, param_tokens;   /* as in pkv_quantize */
    uint8_t* stream; int64_t stream_seq_stride, capacity;
    uint32_t* block_info; int64_t info_seq_stride; uint32_t* stream_bytes;
    uint32_t* flags;
    int32_t batch, heads, tokens, first_token;
    int32_t qblock;                 /* tokens per quantisation block */
    int32_t cb;                     /* tokens per stream block */
    int32_t which;                  /* 0 = K layout, 1 = V layout */
    int32_t bits, mode, high_precision_zero, is_bf16;
    float rel;
} pkv_encode_args;

int32_t pkv_encode_tensor(const pkv_encode_args* args_host, uint8_t* codes_scratch, int64_t scratch_bytes,
                          void* cuda_stream);

/*
 * The same single pass with the reference's median reorder inside (median_repacking, utils/compute.py:262-270:
 * the tokens of every block are sorted by the descending lower median of their V codes, one order for K and V).
 * pkv_value_median_order computes the order straight from fp16/bf16 V (args: x, strides, batch, heads <= 8,
 * tokens, rel, is_bf16 of the V tensor; block = 64): order (batch, tokens/block, block) uint8, entry r = source
 * row of stored row r, stable on ties, per sequence.  pkv_encode_tensor_ordered then encodes K or V reading
 * its rows through that order (per-token parameters land at the stored positions); streams and parameters
 * equal pkv_quantize -> pkv_gather_rows / pkv_gather_params -> pkv_{k,v}_encode.  Restrictions: the modes the
 * single pass serves (K per channel with cb = qblock = order_block, or per token; V per token; no
 * high-precision zero), order_block a multiple of 16 that divides cb; PKV_ERR_UNSUPPORTED otherwise.
 * scratch: 16-byte aligned, at least batch*tokens*heads*128 bytes is always enough.
 */
int32_t pkv_value_median_order(const pkv_encode_args* v_args_host, uint8_t* order, int32_t block, void* cuda_stream);
int32_t pkv_encode_tensor_ordered(const pkv_encode_args* args_host, const uint8_t* order, int32_t order_block,
                                  uint8_t* scratch, int64_t scratch_bytes, void* cuda_stream);

/*
 * pkv_encode_tensor without a scratch argument, for callers that must not touch the device
 * allocator.  (No counterpart in the reference, which allocates freely through torch.)
 *
 * Who needs it: the cache's append step when it runs inside a serving engine's decode loop.  Such
 * engines hand all free HBM to their own KV-block pool at start-up, so a cudaMalloc made later can
 * simply fail, and one that succeeds still stalls the whole device while the driver maps memory --
 * in the middle of a latency-critical step.  They want every per-step call to bring its own memory.
 *
 * The uint8 codes live in a 16 MiB array inside the library image instead
 * (PKV_STATIC_SCRATCH_BYTES; every GPU that loads the library keeps its copy until the process
 * exits).  A call needs batch*tokens*heads*128 bytes of it -- e.g. one 64-token block of 8 KV heads
 * for 256 sequences -- and is refused with PKV_ERR_TOO_LARGE beyond that; use pkv_encode_tensor
 * with your own scratch for bulk prefill.  The call itself allocates nothing and frees nothing.
 *
 * The first call on each device looks up the array's device address (with that device current);
 * make that first call outside any stream capture.  All calls share the one array, which keeps
 * whatever the previous call left in it: this entry point overwrites every byte it later reads, so
 * nothing has to be cleared, but two calls that overlap on the GPU (different streams, or
 * different host threads on one device) race on it -- serialise them.
 * Inputs, outputs and results are exactly those of pkv_encode_tensor.
 */
#define PKV_STATIC_SCRATCH_BYTES (16u << 20)
int32_t pkv_encode_tensor_static(const pkv_encode_args* args_host, void* cuda_stream);

/*
 * Rotary embedding of new K tokens inside the cache; replaces apply_rotary_pos_emb_single
 * (utils/compute.py:32-43) bit for bit.  x/out (batch, heads, tokens, dim <= 128), cos/sin
 * (batch or 1, tokens, dim) with cs_stride_b = 0 to broadcast; strides in elements.
 */
int32_t pkv_rope(const void* x, int64_t x_stride_b, int64_t x_stride_h, int64_t x_stride_s, const void* cos,
                 const void* sin, int64_t cs_stride_b, void* out, int64_t o_stride_b, int64_t o_stride_h,
                 int64_t o_stride_s, int32_t batch, int32_t heads, int32_t tokens, int32_t dim, int32_t is_bf16,
                 void* cuda_stream);

/*
 * Dense reconstruction of quantised tokens, (code + zero) * scale or code * scale + min with the
 * reference's roundings (utils/compute.py:173-178).  codes (batch, tokens, heads*128) as written
 * by pkv_quantize / pkv_{k,v}_decode; scale/zero laid out as in pkv_quantize, the first token of
 * `codes` being token `first_token` of the sequence.  out (batch, heads, tokens, 128).
 */
int32_t pkv_dequantize(const uint8_t* codes, int64_t codes_seq_stride, const void* scale, const void* zero,
                       int32_t param_blocks, int32_t param_tokens, int32_t first_token, void* out,
                       int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int32_t batch, int32_t heads,
                       int32_t tokens, int32_t block, int32_t mode, int32_t high_precision_zero, int32_t is_bf16,
                       void* cuda_stream);

/*
 * Fused decompress-attention decode: out = softmax(q K^T * scaling) V for ONE new query token
 * per sequence over (compressed tokens + uncompressed residual tokens), reading the packed
 * streams directly.  Replaces the chain kq_mat_vec_mul -> fused_kq -> torch softmax ->
 * wv_mat_vec_mul -> fused_wv (packkv_cuda_ext/src/kernels.cu:611-630,842-859,
 * src/fused_kernels.cu:171-185,355-369, evaluation/evaluation.py:1040-1049) and, for the
 * model path, dequantise + eager attention (models/cache/packkv_quant.py:45-85,
 * models/llama.py:177-212), whose rounding points it reproduces.
 *
 * Head dimension is 128.  group = q heads per KV head (1..8).  Element type fp16 or bf16.
 * K quantisation: PKV_K_CHANNEL (scale/zero per (kv head, token block, channel), the
 * reference's QuantMode.ChannelQuant; requires the scale block = cbk) or PKV_K_TOKEN (per
 * token across all heads, QuantMode.TokenQuant).  V quantisation: per token.
 * Streams and their per-sequence strides/capacities must be 16-byte aligned / multiples of
 * 16; n_comp must be a multiple of 128 (64 when cbk = cbv = 64).
 * One thread-block cluster works on each (sequence, KV head); no scratch memory is needed.
 */
typedef struct pkv_attn_args {
    const void* q;              /* (batch, kv_heads*group, 128) */
    void* out;                  /* (batch, kv_heads*group, 128) */
    const uint8_t* k_stream; int64_t k_seq_stride; int64_t k_capacity;
    const uint32_t* k_info;  int64_t k_info_seq_stride;   /* block = ctx_blk*kv_heads + head */
    const void* k_scale; const void* k_zero;              /* channel: (batch, kv_heads, param_blocks, 128); token: (batch, param_tokens) */
    const uint8_t* v_stream; int64_t v_seq_stride; int64_t v_capacity;
    const uint32_t* v_info;  int64_t v_info_seq_stride;   /* block = ctx_blk*2*kv_heads + 2*head + half */
    const void* v_scale; const void* v_zero;              /* (batch, param_tokens) */
    int32_t param_blocks, param_tokens;                   /* row lengths of the parameter arrays (>= n_comp/cbk, >= n_comp) */
    const void* k_res; const void* v_res;                 /* (batch, kv_heads, res_capacity, 128); first n_res tokens valid */
    int64_t res_seq_stride, res_head_stride;              /* in elements */
    int32_t n_res;
    int32_t batch, kv_heads, group;
    int32_t n_comp;
    int32_t cbk, cbv, bits_k, bits_v;
    int32_t k_mode;
    int32_t high_precision_zero;                          /* dequantise as code*scale + min (utils/compute.py:175) */
    int32_t is_bf16;
    float scaling;
    uint32_t* flags;                                      /* device status word */
} pkv_attn_args;

/* `args` is a HOST pointer to the argument block (copied at call time). */
int32_t pkv_decode_attention(const pkv_attn_args* args_host, void* cuda_stream);

/*
 * KV-head-sharded decode over several GPUs of one node (one process per GPU, rank r owns kv_heads local KV
 * heads and their q heads): the same launch, whose last stage also delivers this rank's output rows to every
 * rank.  No counterpart in the reference (it has no multi-GPU path for one sequence).
 *
 * Every rank owns a gathered buffer (n_ranks, batch, kv_heads*group, 128) and an array of n_ranks arrival
 * counters (uint32, zero before the first step), both mapped into the other ranks' address spaces (CUDA IPC
 * or another peer mapping).  gathered[p] / arrivals[p] are rank p's buffers as THIS process addresses them
 * (entry `rank` = this rank's own).  The block that finishes a (sequence, KV head) pair stores its rows into
 * slice `rank` of every gathered[p] with ordinary stores, fences, and adds 1 to arrivals[p][rank]: after a step
 * each counter has grown by batch*kv_heads.  Plain peer stores only: no multicast, no loads from peer memory.
 * args.out still receives the local rows.
 *
 * pkv_exchange_wait makes the stream wait until every arrivals[r] (this rank's own counters) has reached
 * `expected` (compared modulo 2^32): one warp polls with acquire loads for at most `max_polls` rounds a quarter
 * of a microsecond apart and then gives up, setting PKV_FLAG_TIMEOUT in dev_flags (the kernel always returns, so a
 * rank that never arrives costs the others a bounded wait, not a hang).  Kernels after it on the stream see the
 * gathered rows.  A rank must not start step s+2 into the same gathered buffer before it has waited for step
 * s+1: alternate two buffers per layer or wait every step.
 */
typedef struct pkv_attn_exchange {
    int32_t n_ranks;            /* 1..8 */
    int32_t rank;
    void* gathered[8];
    uint32_t* arrivals[8];
} pkv_attn_exchange;
int32_t pkv_decode_attention_exchange(const pkv_attn_args* args_host, const pkv_attn_exchange* exchange_host,
                                      void* cuda_stream);
int32_t pkv_exchange_wait(const uint32_t* arrivals, int32_t n_ranks, uint32_t expected, uint32_t max_polls,
                          uint32_t* dev_flags, void* cuda_stream);
/*
 * The same wait, but once every counter has reached per_step (the arrivals of ONE step: batch * local KV heads) that
 * many are taken off it again.  The call is then identical for every step, so a CUDA graph that holds the layer loop
 * (attention launches with their exchange blocks and these waits) can be replayed step after step.  With two
 * alternating buffer / counter sets a peer's arrivals for step s + 2 cannot reach a counter before this rank has
 * taken step s off it: the peer starts s + 2 only after it has seen this rank's step s + 1, which this rank's stream
 * launches after this wait.
 */
int32_t pkv_exchange_wait_consume(uint32_t* arrivals, int32_t n_ranks, uint32_t per_step, uint32_t max_polls,
                                  uint32_t* dev_flags, void* cuda_stream);
/*
 * Decode step with the append folded in: the launch first writes the step's new token (K after RoPE with the
 * arithmetic of pkv_rope, V as is) into row n_res-1 of the residual buffers and then attends over all n_res
 * residual tokens, i.e. args.n_res COUNTS the new token.  Replaces the pair
 * past_key_value.update(...) + attention of a decode step (models/llama.py:259-282,
 * models/cache/packkv_quant.py:57-60) when no block leaves the residual in this step; saves the separate
 * pkv_append_residual launch.  new_k / new_v: (batch, kv_heads, 1, 128), strides in elements; cos / sin:
 * (batch or 1, 1, 128) with cs_stride_b = 0 for a shared row, or both NULL if new_k is already rotated.
 * res_capacity = rows of the residual buffers (n_res <= res_capacity is checked).  `exchange_host` may be NULL.
 */
typedef struct pkv_attn_append {
    const void* new_k; const void* new_v;
    int64_t k_stride_b, k_stride_h, v_stride_b, v_stride_h;
    const void* cos; const void* sin;
    int64_t cs_stride_b;
    int32_t res_capacity;
} pkv_attn_append;
int32_t pkv_decode_attention_append(const pkv_attn_args* args_host, const pkv_attn_append* append_host,
                                    const pkv_attn_exchange* exchange_host, void* cuda_stream);

/*
 * Decode attention with a work split the caller can see and steer, for launches with few (sequence, KV head)
 * pairs (batch 1-2 at long contexts, the regime of scripts/rebuttal_throughout.py:28-37, or KV heads sharded
 * over many GPUs), where one cluster of at most 16 CTAs per pair leaves most of the GPU idle.  With `scratch`
 * the library may run the step as TWO launches with `nsplit` clusters per pair: the first computes the scores
 * of all tokens (K phase) and leaves them, with every CTA's maximum and sum, in the scratch; the second
 * normalises with the global maximum and sum, rounds the probabilities, contracts V, and the pair's last
 * cluster to finish adds the clusters' rows in a fixed order.  Rounding points are those of the single launch.
 *   plan_io   in: cluster (CTAs per cluster, 1..16), nsplit (clusters per pair), launches (1 or 2), extra to force,
 *             0 = let the library choose; out: what was used.  May be NULL.  Without an exchange block the library may
 *             give the pairs unequal numbers of CTAs (`extra` > 0) when that fills the GPU better.  Two launches of the same tensors with
 *             the same cluster * nsplit give bit-identical results whatever the batch and head counts.
 *   scratch   device memory, 256-byte aligned, ZERO before its first use (the library leaves its counters at
 *             zero after every call); launches that share it must be ordered on one stream.  NULL: single launch.
 * pkv_attention_plan fills plan_io the same way and launches nothing (scratch_bytes alone decides what fits;
 * with_exchange != 0: plan as for a launch with an exchange block).
 * append_host and exchange_host may be NULL.
 */
typedef struct pkv_attn_plan {
    int32_t cluster;
    int32_t nsplit;
    int32_t launches;
    int32_t extra;      /* two launches with cluster 1: the first `extra` pairs get nsplit + 1 CTAs, the others nsplit,
                           so that all pairs' CTAs together fill the GPU's CTA slots exactly; 0 = the same for all */
} pkv_attn_plan;
int32_t pkv_decode_attention_split(const pkv_attn_args* args_host, const pkv_attn_append* append_host,
                                   const pkv_attn_exchange* exchange_host, pkv_attn_plan* plan_io,
                                   void* scratch, int64_t scratch_bytes, void* cuda_stream);
int32_t pkv_attention_plan(const pkv_attn_args* args_host, pkv_attn_plan* plan_io, int64_t scratch_bytes,
                           int32_t with_exchange);

/*
 * Set-up helpers of the exchange; the only entry points that allocate or touch address-space mappings (they
 * synchronise, call them once, outside the decode loop).  pkv_exchange_alloc returns `bytes` of zeroed device
 * memory on the current device (its own cudaMalloc, so that it can be exported) and the 64-byte
 * cudaIpcMemHandle that another process of the node passes to pkv_ipc_open, which maps the buffer into the
 * CURRENT device's address space with peer access to the owning GPU, so that this device's kernels can store
 * into it.  pkv_ipc_close unmaps, pkv_exchange_free releases.
 */
int32_t pkv_exchange_alloc(int64_t bytes, void** ptr_host, uint8_t* handle64_host);
int32_t pkv_exchange_free(void* ptr);
int32_t pkv_ipc_open(const uint8_t* handle64_host, void** mapped_host);
int32_t pkv_ipc_close(void* mapped);

#ifdef __cplusplus
}
#endif
#endif /* PACKKV_SM100_H */
