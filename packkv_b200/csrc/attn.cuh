// Host-side interface of the fused decompress-attention decode kernel.  The argument block
// is the C ABI's pkv_attn_args (include/packkv_sm100.h); all pointers are device pointers.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include "../../include/packkv_sm100.h"

namespace pkv {

enum KMode : int { kKChannel = PKV_K_CHANNEL, kKToken = PKV_K_TOKEN };
using AttnArgs = pkv_attn_args;

using AttnExchange = pkv_attn_exchange;
using AttnAppend = pkv_attn_append;
using AttnPlan = pkv_attn_plan;

// xch may be null (single GPU); ap may be null (the residual already holds every token); plan_io may be null
// (choose everything); scratch may be null (single-launch form only); dry_run: fill plan_io, launch nothing
int launch_attention(const AttnArgs& a, const AttnExchange* xch, const AttnAppend* ap, AttnPlan* plan_io, void* scratch, int64_t scratch_bytes,
                     bool dry_run, cudaStream_t st);
int launch_exchange_wait(uint32_t* arrivals, int n_ranks, unsigned expected, unsigned max_polls, unsigned* flags, bool consume, cudaStream_t st);

}  // namespace pkv
