// extern "C" surface of libpackkv_sm100.so; declarations and contracts live in
// include/packkv_sm100.h.
#include <cstring>
#include "../../include/packkv_sm100.h"
#include "common.cuh"
#include "launch.h"
#include "attn.cuh"

using namespace pkv;

extern "C" {

int32_t pkv_abi_version(void) { return 1; }

static int32_t codec_call(bool is_k, bool encode, const uint8_t* codes, int64_t codes_seq_stride, uint8_t* stream,
                          int64_t stream_seq_stride, int64_t capacity, uint32_t* info, int64_t info_seq_stride,
                          uint32_t* stream_bytes, uint32_t* flags, int32_t n_seq, int32_t ctx_len, int32_t hidden,
                          int32_t cb, int32_t hb, int32_t bits, int32_t first_cb, void* cuda_stream) {
    CodecShape sh{n_seq, ctx_len, hidden, cb, hb, bits, first_cb};
    CodecBuffers b{codes, codes_seq_stride, stream, stream_seq_stride, capacity, info, info_seq_stride, stream_bytes, flags};
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    return encode ? launch_encode(is_k, sh, b, st) : launch_decode(is_k, sh, b, st);
}

int32_t pkv_k_encode(const uint8_t* codes, int64_t codes_seq_stride, uint8_t* stream, int64_t stream_seq_stride,
                     int64_t capacity, uint32_t* block_info, int64_t info_seq_stride, uint32_t* stream_bytes,
                     uint32_t* dev_flags, int32_t n_seq, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb,
                     int32_t bits, int32_t first_cb, void* cuda_stream) {
    return codec_call(true, true, codes, codes_seq_stride, stream, stream_seq_stride, capacity, block_info, info_seq_stride,
                      stream_bytes, dev_flags, n_seq, ctx_len, hidden, cb, hb, bits, first_cb, cuda_stream);
}

int32_t pkv_v_encode(const uint8_t* codes, int64_t codes_seq_stride, uint8_t* stream, int64_t stream_seq_stride,
                     int64_t capacity, uint32_t* block_info, int64_t info_seq_stride, uint32_t* stream_bytes,
                     uint32_t* dev_flags, int32_t n_seq, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb,
                     int32_t bits, int32_t first_cb, void* cuda_stream) {
    return codec_call(false, true, codes, codes_seq_stride, stream, stream_seq_stride, capacity, block_info, info_seq_stride,
                      stream_bytes, dev_flags, n_seq, ctx_len, hidden, cb, hb, bits, first_cb, cuda_stream);
}

int32_t pkv_k_decode(const uint8_t* stream, int64_t stream_seq_stride, int64_t capacity, const uint32_t* block_info,
                     int64_t info_seq_stride, uint8_t* codes, int64_t codes_seq_stride, uint32_t* dev_flags,
                     int32_t n_seq, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb, int32_t bits,
                     int32_t first_cb, void* cuda_stream) {
    return codec_call(true, false, codes, codes_seq_stride, const_cast<uint8_t*>(stream), stream_seq_stride, capacity,
                      const_cast<uint32_t*>(block_info), info_seq_stride, nullptr, dev_flags, n_seq, ctx_len, hidden, cb, hb,
                      bits, first_cb, cuda_stream);
}

int32_t pkv_v_decode(const uint8_t* stream, int64_t stream_seq_stride, int64_t capacity, const uint32_t* block_info,
                     int64_t info_seq_stride, uint8_t* codes, int64_t codes_seq_stride, uint32_t* dev_flags,
                     int32_t n_seq, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb, int32_t bits,
                     int32_t first_cb, void* cuda_stream) {
    return codec_call(false, false, codes, codes_seq_stride, const_cast<uint8_t*>(stream), stream_seq_stride, capacity,
                      const_cast<uint32_t*>(block_info), info_seq_stride, nullptr, dev_flags, n_seq, ctx_len, hidden, cb, hb,
                      bits, first_cb, cuda_stream);
}

int32_t pkv_kq_mat_vec_mul(const uint8_t* stream, int64_t stream_bytes, const uint32_t* block_info, const void* q,
                           void* kq_out, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb, int32_t bits,
                           int32_t is_bf16, uint32_t* dev_flags, void* cuda_stream) {
    LegacyArgs a{stream, stream_bytes, block_info, q, kq_out, ctx_len, hidden, cb, hb, bits, is_bf16, dev_flags};
    return launch_legacy_matvec(true, a, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_wv_mat_vec_mul(const uint8_t* stream, int64_t stream_bytes, const uint32_t* block_info, const void* w,
                           float* wv_out, int32_t ctx_len, int32_t hidden, int32_t cb, int32_t hb, int32_t bits,
                           int32_t is_bf16, uint32_t* dev_flags, void* cuda_stream) {
    LegacyArgs a{stream, stream_bytes, block_info, w, wv_out, ctx_len, hidden, cb, hb, bits, is_bf16, dev_flags};
    return launch_legacy_matvec(false, a, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_fused_kq(void* our_kq, const void* q, const void* zero, const void* scale, const void* t, int32_t M,
                     int32_t N, int32_t K, int32_t is_bf16, void* cuda_stream) {
    return launch_fused_epilogue(true, our_kq, q, zero, scale, t, M, N, K, is_bf16, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_fused_wv(void* our_wv, const void* w, const void* zero, const void* scale, const void* term1, int32_t M,
                     int32_t N, int32_t D, int32_t is_bf16, void* cuda_stream) {
    return launch_fused_epilogue(false, our_wv, w, zero, scale, term1, M, N, D, is_bf16, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_quantize(const void* x, int64_t stride_b, int64_t stride_h, int64_t stride_s, uint8_t* codes,
                     int64_t codes_seq_stride, void* scale, void* zero, int32_t param_blocks, int32_t first_block,
                     int32_t param_tokens, int32_t first_token, int32_t batch, int32_t heads, int32_t tokens,
                     int32_t block, float rel, int32_t bits, int32_t mode, int32_t high_precision_zero,
                     int32_t is_bf16, uint32_t* dev_flags, void* cuda_stream) {
    QuantArgs q{x, stride_b, stride_h, stride_s, codes, codes_seq_stride, scale, zero, param_blocks, first_block,
                param_tokens, first_token, batch, heads, tokens, block, rel, bits, mode, high_precision_zero, is_bf16, dev_flags};
    return launch_quantize(q, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_median_order(const uint8_t* v_codes, int64_t codes_seq_stride, uint8_t* order, uint8_t* keys,
                         int32_t batch, int32_t heads, int32_t tokens, int32_t block, void* cuda_stream) {
    ReorderArgs a{v_codes, codes_seq_stride, order, keys, batch, heads, tokens, block};
    return launch_median_order(a, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_gather_rows(const uint8_t* src, uint8_t* dst, int64_t seq_stride, const uint8_t* order, int32_t batch,
                        int32_t tokens, int32_t block, int32_t row_bytes, void* cuda_stream) {
    return launch_gather_rows(src, dst, seq_stride, order, batch, tokens, block, row_bytes, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_gather_params(const void* src, void* dst, int64_t row_len, int32_t first, const uint8_t* order,
                          int32_t batch, int32_t tokens, int32_t block, void* cuda_stream) {
    return launch_gather_params(src, dst, row_len, first, order, batch, tokens, block, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_append_residual(const void* k, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s, const void* v,
                            int64_t v_stride_b, int64_t v_stride_h, int64_t v_stride_s, const void* cos, const void* sin,
                            int64_t cs_stride_b, void* k_res, void* v_res, int64_t res_stride_b, int64_t res_stride_h,
                            int32_t res_capacity, int32_t position, int32_t batch, int32_t heads, int32_t tokens,
                            int32_t is_bf16, void* cuda_stream) {
    AppendArgs r{k, k_stride_b, k_stride_h, k_stride_s, v, v_stride_b, v_stride_h, v_stride_s, cos, sin, cs_stride_b,
                 k_res, v_res, res_stride_b, res_stride_h, res_capacity, position, batch, heads, tokens, is_bf16};
    return launch_append(r, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_greedy_order(const uint8_t* k_codes, const uint8_t* v_codes, int64_t codes_seq_stride, uint8_t* order,
                         int32_t batch, int32_t heads, int32_t tokens, int32_t block, int32_t pack_len, void* cuda_stream) {
    return launch_greedy_order(k_codes, v_codes, codes_seq_stride, order, batch, heads, tokens, block, pack_len,
                               static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_size_model(const uint8_t* codes, int64_t codes_seq_stride, int32_t batch, int32_t tokens, int32_t hidden,
                       int32_t pack_len, uint64_t* bits_sum, uint32_t* present, void* cuda_stream) {
    return launch_size_model(codes, codes_seq_stride, batch, tokens, hidden, pack_len,
                             reinterpret_cast<unsigned long long*>(bits_sum), present, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_rope(const void* x, int64_t x_stride_b, int64_t x_stride_h, int64_t x_stride_s, const void* cos,
                 const void* sin, int64_t cs_stride_b, void* out, int64_t o_stride_b, int64_t o_stride_h,
                 int64_t o_stride_s, int32_t batch, int32_t heads, int32_t tokens, int32_t dim, int32_t is_bf16,
                 void* cuda_stream) {
    RopeArgs r{x, x_stride_b, x_stride_h, x_stride_s, cos, sin, cs_stride_b, out, o_stride_b, o_stride_h, o_stride_s,
               batch, heads, tokens, dim, is_bf16};
    return launch_rope(r, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_dequantize(const uint8_t* codes, int64_t codes_seq_stride, const void* scale, const void* zero,
                       int32_t param_blocks, int32_t param_tokens, int32_t first_token, void* out,
                       int64_t o_stride_b, int64_t o_stride_h, int64_t o_stride_s, int32_t batch, int32_t heads,
                       int32_t tokens, int32_t block, int32_t mode, int32_t high_precision_zero, int32_t is_bf16,
                       void* cuda_stream) {
    DequantArgs q{codes, codes_seq_stride, scale, zero, param_blocks, param_tokens, first_token, out, o_stride_b,
                  o_stride_h, o_stride_s, batch, heads, tokens, block, mode, high_precision_zero, is_bf16};
    return launch_dequantize(q, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_decode_attention(const pkv_attn_args* args_host, void* cuda_stream) {
    if (!args_host) return kBadArgument;
    return launch_attention(*args_host, nullptr, nullptr, nullptr, nullptr, 0, false, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_decode_attention_exchange(const pkv_attn_args* args_host, const pkv_attn_exchange* exchange_host, void* cuda_stream) {
    if (!args_host || !exchange_host) return kBadArgument;
    return launch_attention(*args_host, exchange_host, nullptr, nullptr, nullptr, 0, false, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_decode_attention_append(const pkv_attn_args* args_host, const pkv_attn_append* append_host, const pkv_attn_exchange* exchange_host,
                                    void* cuda_stream) {
    if (!args_host || !append_host) return kBadArgument;
    return launch_attention(*args_host, exchange_host, append_host, nullptr, nullptr, 0, false, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_decode_attention_split(const pkv_attn_args* args_host, const pkv_attn_append* append_host, const pkv_attn_exchange* exchange_host,
                                   pkv_attn_plan* plan_io, void* scratch, int64_t scratch_bytes, void* cuda_stream) {
    if (!args_host) return kBadArgument;
    return launch_attention(*args_host, exchange_host, append_host, plan_io, scratch, scratch_bytes, false, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_attention_plan(const pkv_attn_args* args_host, pkv_attn_plan* plan_io, int64_t scratch_bytes, int32_t with_exchange) {
    if (!args_host || !plan_io) return kBadArgument;
    // the plan depends on sizes only: any non-null, aligned address stands for the scratch, and a block that is never
    // dereferenced (nothing is launched) for the exchange
    pkv_attn_exchange x{};
    x.n_ranks = 1;
    uint32_t dummy_counter = 0;
    x.gathered[0] = &dummy_counter; x.arrivals[0] = &dummy_counter;
    return launch_attention(*args_host, with_exchange ? &x : nullptr, nullptr, plan_io, scratch_bytes > 0 ? reinterpret_cast<void*>(uintptr_t(256)) : nullptr,
                            scratch_bytes, true, nullptr);
}

int32_t pkv_exchange_wait(const uint32_t* arrivals, int32_t n_ranks, uint32_t expected, uint32_t max_polls, uint32_t* dev_flags,
                          void* cuda_stream) {
    return launch_exchange_wait(const_cast<uint32_t*>(arrivals), n_ranks, expected, max_polls, dev_flags, false, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_exchange_wait_consume(uint32_t* arrivals, int32_t n_ranks, uint32_t per_step, uint32_t max_polls, uint32_t* dev_flags,
                                  void* cuda_stream) {
    return launch_exchange_wait(arrivals, n_ranks, per_step, max_polls, dev_flags, true, static_cast<cudaStream_t>(cuda_stream));
}

int32_t pkv_exchange_alloc(int64_t bytes, void** ptr_host, uint8_t* handle64_host) {
    if (bytes <= 0 || !ptr_host || !handle64_host) return kBadArgument;
    void* p = nullptr;
    if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) { cudaGetLastError(); return kCudaError; }
    cudaIpcMemHandle_t h;
    if (cudaMemset(p, 0, (size_t)bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(p);
        return kCudaError;
    }
    memcpy(handle64_host, &h, sizeof(h));
    *ptr_host = p;
    return kOk;
}

int32_t pkv_exchange_free(void* ptr) {
    if (!ptr) return kBadArgument;
    return cudaFree(ptr) == cudaSuccess ? kOk : kCudaError;
}

int32_t pkv_ipc_open(const uint8_t* handle64_host, void** mapped_base_host) {
    if (!handle64_host || !mapped_base_host) return kBadArgument;
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
    memcpy(&h, handle64_host, sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return kCudaError; }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
        cudaGetLastError();
        cudaIpcCloseMemHandle(p);
        return kCudaError;
    }
    *mapped_base_host = p;
    return kOk;
}

int32_t pkv_ipc_close(void* mapped_base) {
    if (!mapped_base) return kBadArgument;
    return cudaIpcCloseMemHandle(mapped_base) == cudaSuccess ? kOk : kCudaError;
}

}  // extern "C"
