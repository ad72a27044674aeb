// Host-side launch interfaces shared between the kernel translation units and the C ABI.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "../../include/packkv_sm100.h"

namespace pkv {

struct CodecShape {
    int n_seq;       // independent sequences (each has its own stream and block_info rows)
    int ctx_len;     // tokens in this call (multiple of cb)
    int hidden;      // channels per token row (multiple of hb)
    int cb, hb;      // block shape: tokens x channels (K: hb 128, V: hb 64)
    int bits;        // 2, 3 or 4
    int first_cb;    // index of the first token block of this call inside the sequence
};

struct CodecBuffers {
    const uint8_t* codes;       // encode: input; decode: output (cast away const by the callee)
    int64_t codes_seq_stride;   // bytes between sequences
    uint8_t* stream;
    int64_t stream_seq_stride;  // bytes between sequences
    int64_t capacity;           // usable bytes of each sequence's stream
    uint32_t* info;             // (offset, size) pairs; rows of sequence s start at s*info_seq_stride
    int64_t info_seq_stride;    // in blocks
    uint32_t* stream_bytes;     // per sequence: bytes used so far (encode: in/out)
    unsigned* flags;            // device status word, OR-ed with DevFlag bits
};

struct QuantArgs {
    const void* x;               // (B, H, S, 128) elements; strides in elements, channels contiguous
    int64_t stride_b, stride_h, stride_s;
    uint8_t* codes;              // (B, S, H*128) uint8
    int64_t codes_seq_stride;    // bytes between sequences
    void* scale; void* zero;     // channel: (B, H, param_blocks, 128); token: (B, param_tokens)
    int param_blocks, first_block;   // channel mode: capacity in blocks, index of this call's first block
    int param_tokens, first_token;   // token mode: capacity in tokens, index of this call's first token
    int batch, heads, tokens, block;
    float rel;
    int bits;                    // 0 = do not range-check the codes
    int mode;                    // 0 = channel, 1 = token
    int high_precision_zero;
    int is_bf16;
    unsigned* flags;
};

struct LegacyArgs {
    const uint8_t* stream; int64_t stream_bytes;   // one sequence; valid bytes
    const uint32_t* info;
    const void* vec;      // kq: q (hidden/128, 128) lane-permuted; wv: w (hidden/128, ctx_len)
    void* out;            // kq: (hidden/128, ctx_len) element type; wv: (hidden) float, accumulated into
    int ctx_len, hidden, cb, hb, bits, is_bf16;
    unsigned* flags;
};

int launch_legacy_matvec(bool is_k, const LegacyArgs& a, cudaStream_t st);
int launch_fused_epilogue(bool is_kq, void* out, const void* a, const void* zero, const void* scale, const void* t,
                          int M, int N, int K, int is_bf16, cudaStream_t st);
struct RopeArgs {
    const void* x; int64_t x_stride_b, x_stride_h, x_stride_s;   // (B, H, T, dim), strides in elements
    const void* cos; const void* sin; int64_t cs_stride_b;       // (B or 1, T, dim); cs_stride_b = 0 broadcasts
    void* out; int64_t o_stride_b, o_stride_h, o_stride_s;
    int batch, heads, tokens, dim, is_bf16;
};
struct AppendArgs {
    const void* k; int64_t k_stride_b, k_stride_h, k_stride_s;   // new K (B, H, T, 128), strides in elements
    const void* v; int64_t v_stride_b, v_stride_h, v_stride_s;   // new V
    const void* cos; const void* sin; int64_t cs_stride_b;       // (B or 1, T, 128) or both null: K is already rotated
    void* k_res; void* v_res; int64_t res_stride_b, res_stride_h; // residual buffers (B, H, capacity, 128)
    int res_capacity, position;                                    // rows [position, position + tokens) are written
    int batch, heads, tokens, is_bf16;
};
struct DequantArgs {
    const uint8_t* codes; int64_t codes_seq_stride;               // (B, T, H*128)
    const void* scale; const void* zero;
    int param_blocks, param_tokens, first_token;                  // layout of scale/zero as in QuantArgs
    void* out; int64_t o_stride_b, o_stride_h, o_stride_s;         // (B, H, T, 128), strides in elements
    int batch, heads, tokens, block, mode, high_precision_zero, is_bf16;
};
struct ReorderArgs {
    const uint8_t* v_codes; int64_t codes_seq_stride;   // (B, tokens, heads*128) uint8
    uint8_t* order;                                     // (B, tokens/block, block): source row of each rank
    uint8_t* keys;                                      // optional (B, tokens): the per-token median
    int batch, heads, tokens, block;
};
int launch_median_order(const ReorderArgs& a, cudaStream_t st);
int launch_greedy_order(const uint8_t* k_codes, const uint8_t* v_codes, int64_t seq_stride, uint8_t* order, int batch, int heads,
                        int tokens, int block, int pack_len, cudaStream_t st);
int launch_size_model(const uint8_t* codes, int64_t seq_stride, int batch, int tokens, int hidden, int pack_len,
                      unsigned long long* bits_sum, unsigned* present, cudaStream_t st);
int launch_gather_rows(const uint8_t* src, uint8_t* dst, int64_t seq_stride, const uint8_t* order, int batch, int tokens,
                       int block, int row_bytes, cudaStream_t st);
int launch_gather_params(const void* src, void* dst, int64_t row_len, int first, const uint8_t* order, int batch, int tokens,
                         int block, cudaStream_t st);
int launch_rope(const RopeArgs& r, cudaStream_t st);
int launch_append(const AppendArgs& r, cudaStream_t st);
int launch_dequantize(const DequantArgs& q, cudaStream_t st);
int launch_quantize(const QuantArgs& q, cudaStream_t st);
// single-pass encoder (fused_encode.cu); the request is the C ABI's argument block
using FusedEncodeRequest = pkv_encode_args;
bool fused_encode_applicable(const FusedEncodeRequest& r);
int64_t fused_encode_scratch_bytes(const FusedEncodeRequest& r);
// order (optional): (batch, tokens / order_block, order_block) uint8, source row of every stored row of a reorder block
int launch_fused_encode(const FusedEncodeRequest& r, uint8_t* slots, const uint8_t* order, int order_block, cudaStream_t st);
// token order of every `block` tokens by descending lower median of the V codes, straight from fp16/bf16 V
int launch_value_median_order(const FusedEncodeRequest& r, uint8_t* order, int block, cudaStream_t st);
int launch_scan_sizes(const CodecShape& sh, const CodecBuffers& b, cudaStream_t st);
int launch_encode(bool is_k, const CodecShape& sh, const CodecBuffers& b, cudaStream_t st);
int launch_decode(bool is_k, const CodecShape& sh, const CodecBuffers& b, cudaStream_t st);

}  // namespace pkv
