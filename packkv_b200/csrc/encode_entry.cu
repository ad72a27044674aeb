// One-call encoder entry point: quantise fp16/bf16 K or V and bit-pack the codes into the
// per-sequence streams (pkv_quantize followed by pkv_{k,v}_encode on a scratch code matrix).
#include <mutex>

#include "../../include/packkv_sm100.h"
#include "common.cuh"
#include "launch.h"

using namespace pkv;

// Scratch of the allocation-free entry point: lives in the library image, one copy per GPU that
// loads the library, held until the process exits.
static __device__ __align__(256) uint8_t g_static_codes[PKV_STATIC_SCRATCH_BYTES];

static int32_t encode_tensor(const pkv_encode_args& e, uint8_t* codes, cudaStream_t st) {
    if (e.which != 0 && e.which != 1) return kBadArgument;
    if (e.cb <= 0 || e.first_token % e.cb) return kBadArgument;
    // K per-channel and V per-token go through the single-pass kernels; the scratch then holds
    // fixed-stride block slots (smaller than the code matrix it is sized for)
    if (fused_encode_applicable(e) && fused_encode_scratch_bytes(e) <= (int64_t)e.batch * e.tokens * e.heads * 128)
        return launch_fused_encode(e, codes, nullptr, 0, st);
    QuantArgs q{e.x, e.stride_b, e.stride_h, e.stride_s, codes, (int64_t)e.tokens * e.heads * 128, e.scale, e.zero,
                e.param_blocks, e.qblock > 0 ? e.first_token / e.qblock : 0, e.param_tokens, e.first_token,
                e.batch, e.heads, e.tokens, e.qblock, e.rel, e.bits, e.mode, e.high_precision_zero, e.is_bf16, e.flags};
    int rc = launch_quantize(q, st);
    if (rc != kOk) return rc;
    CodecShape sh{e.batch, e.tokens, e.heads * 128, e.cb, e.which == 0 ? 128 : 64, e.bits, e.first_token / e.cb};
    CodecBuffers b{codes, (int64_t)e.tokens * e.heads * 128, e.stream, e.stream_seq_stride, e.capacity, e.block_info,
                   e.info_seq_stride, e.stream_bytes, e.flags};
    return launch_encode(e.which == 0, sh, b, st);
}

extern "C" int32_t pkv_encode_tensor(const pkv_encode_args* args_host, uint8_t* codes_scratch, int64_t scratch_bytes,
                                     void* cuda_stream) {
    if (!args_host) return kBadArgument;
    const pkv_encode_args& e = *args_host;
    if (e.batch < 0 || e.heads <= 0 || e.tokens < 0) return kBadArgument;
    const int64_t need = (int64_t)e.batch * e.tokens * e.heads * 128;
    if (need == 0) return kOk;
    if (!codes_scratch || scratch_bytes < need || (reinterpret_cast<uintptr_t>(codes_scratch) & 15)) return kBadArgument;
    return encode_tensor(e, codes_scratch, static_cast<cudaStream_t>(cuda_stream));
}

extern "C" int32_t pkv_encode_tensor_ordered(const pkv_encode_args* args_host, const uint8_t* order, int32_t order_block, uint8_t* scratch,
                                             int64_t scratch_bytes, void* cuda_stream) {
    if (!args_host || !order) return kBadArgument;
    const pkv_encode_args& e = *args_host;
    if (e.batch < 0 || e.heads <= 0 || e.tokens < 0 || (e.which != 0 && e.which != 1) || e.cb <= 0 || e.first_token % e.cb) return kBadArgument;
    if ((int64_t)e.batch * e.tokens == 0) return kOk;
    if (!fused_encode_applicable(e)) return kUnsupported;
    if (!scratch || scratch_bytes < fused_encode_scratch_bytes(e) || (reinterpret_cast<uintptr_t>(scratch) & 15)) return kBadArgument;
    return launch_fused_encode(e, scratch, order, order_block, static_cast<cudaStream_t>(cuda_stream));
}

extern "C" int32_t pkv_value_median_order(const pkv_encode_args* v_args_host, uint8_t* order, int32_t block, void* cuda_stream) {
    if (!v_args_host) return kBadArgument;
    return launch_value_median_order(*v_args_host, order, block, static_cast<cudaStream_t>(cuda_stream));
}

// Device address of g_static_codes on the current device.  In host code the symbol's name is only
// a handle, never a pointer a kernel may use, so the address is looked up once per device.
static int static_scratch(uint8_t** out) {
    static std::mutex mu;
    static uint8_t* ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kCudaError;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_codes) != cudaSuccess || !p) return kCudaError;
        ptrs[dev] = static_cast<uint8_t*>(p);
    }
    *out = ptrs[dev];
    return kOk;
}

extern "C" int32_t pkv_encode_tensor_static(const pkv_encode_args* args_host, void* cuda_stream) {
    if (!args_host) return kBadArgument;
    const pkv_encode_args& e = *args_host;
    if (e.batch < 0 || e.heads <= 0 || e.tokens < 0) return kBadArgument;
    const int64_t need = (int64_t)e.batch * e.tokens * e.heads * 128;
    if (need == 0) return kOk;
    if (need > (int64_t)PKV_STATIC_SCRATCH_BYTES) return PKV_ERR_TOO_LARGE;
    uint8_t* codes = nullptr;
    const int rc = static_scratch(&codes);
    if (rc != kOk) return rc;
    return encode_tensor(e, codes, static_cast<cudaStream_t>(cuda_stream));
}
