"""Headline benchmark: fused decompress-attention decode over a compressed KV cache.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload llama8b]

Workload (default, N=1): Llama-3.1-8B-shaped decode attention -- 32 layers, 32 q heads / 8 KV
heads, head_dim 128, bf16, batch 16, context 8192 (8064 compressed tokens + 128 uncompressed
residual tokens per the cache's cut rule), K per-channel 4 bit, V per-token 4 bit, block 64.
Synthetic KV (packkv_b200.synth) stands in for real-model caches.  One STEP = one decode step's
attention for all layers = 32 launches of the fused kernel producing `batch` tokens.

Multi-GPU (torchrun, one rank per GPU): sequences are independent, so the batch is sharded with
no data-path collective; every rank holds a full `batch` of sequences (weak scaling) and the
reported value is (all ranks' tokens) / (max over ranks of the device time).

JSON line: metric decode tok/s; `value` with q/out resident in HBM; `e2e` through the public
API with q in pinned host memory and the output read back every layer; `roofline` on the
algorithmic compressed bytes of the fused kernel; `cpu_baseline` = the reference's own CPU path
(C++ bit-unpack + torch dequantise + eager attention) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: layers, batch, q_heads, kv_heads, ctx, dtype, bits_k, bits_v, block, cbk, cbv
    "llama8b": dict(layers=32, batch=16, q_heads=32, kv_heads=8, ctx=8192, dtype="bf16", bits_k=4, bits_v=4,
                    block=64, cbk=64, cbv=64, name="llama-3.1-8b-shaped decode attention, batch 16, ctx 8192, 4-bit K/V, block 64"),
    "qwen8b-long": dict(layers=36, batch=8, q_heads=32, kv_heads=8, ctx=32768, dtype="bf16", bits_k=2, bits_v=4,
                        block=128, cbk=128, cbv=128, name="qwen3-8b-shaped decode attention, batch 8, ctx 32768, 2-bit K / 4-bit V, block 128"),
    "llama8b-2l": dict(layers=2, batch=16, q_heads=32, kv_heads=8, ctx=8192, dtype="bf16", bits_k=4, bits_v=4,
                       block=64, cbk=64, cbv=64, name="2 layers of the llama-3.1-8b-shaped workload (profiling case)"),
    "tiny": dict(layers=2, batch=2, q_heads=8, kv_heads=2, ctx=1024, dtype="bf16", bits_k=4, bits_v=4,
                 block=64, cbk=64, cbv=64, name="tiny smoke workload"),
}
RECENT = 192   # buffer_size of every reference script (128 + 64)

# dram__bytes_read.sum + dram__bytes_write.sum from the ncu captures summarised under profiles/
# (per launch for the attention kernel, per step for the encoder); only captured shapes have an entry
NCU_TRAFFIC_BYTES = {
    ("attn", 16, 8192, 8, 4, 4, 64): 158.5e6,        # profiles/attn_decode_kernel_llama8b.md
    ("mistral7b-encode", 16, 4, 64): 1836e6,          # profiles/fused_encode_kernels_mistral7b.md
}


def split_context(ctx: int, block: int, recent: int = RECENT):
    n_blocks = max(0, (ctx + block - ctx % block - recent) // block)
    return n_blocks * block, ctx - n_blocks * block


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.stop_flag = index, [], False
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            time.sleep(0.1)

    def start(self):
        self.thread.start()

    def stop(self):
        self.stop_flag = True
        self.thread.join(timeout=6)
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
def build_layers(w, device, dtype, head_shard=None):
    from packkv_b200 import encode, parallel, synth
    from packkv_b200.config import QuantMode
    n_comp, n_res = split_context(w["ctx"], w["block"])
    layers = []
    for li in range(w["layers"]):
        k, v = synth.synth_kv(w["batch"], w["kv_heads"], w["ctx"], 128, seed=1000 + li, dtype=dtype, device=device, apply_rope=True)
        kw = dict(block=w["block"], bits_k=w["bits_k"], bits_v=w["bits_v"], k_rel=synth.rel_for_bits(w["bits_k"]),
                  v_rel=synth.rel_for_bits(w["bits_v"]), k_mode=QuantMode.TokenQuant if w.get("k_mode") == "token" else QuantMode.ChannelQuant,
                  cbk=w["cbk"], cbv=w["cbv"])
        if head_shard is None:
            layer = encode.compress_kv(k[:, :, :n_comp], v[:, :, :n_comp], **kw)
        else:
            layer, (lo, hi) = parallel.compress_kv_head_shard(k[:, :, :n_comp], v[:, :, :n_comp], head_shard[0], head_shard[1], **kw)
            k, v = k[:, lo:hi], v[:, lo:hi]
        # trim the streams to what is used (setup only), keeping 16-byte multiples
        kb = (int(layer.k_bytes.max().item()) + 31) // 16 * 16
        vb = (int(layer.v_bytes.max().item()) + 31) // 16 * 16
        layer.k_stream = layer.k_stream[:, :kb].contiguous()
        layer.v_stream = layer.v_stream[:, :vb].contiguous()
        k_res = k[:, :, n_comp:].contiguous()
        v_res = v[:, :, n_comp:].contiguous()
        layers.append((layer, k_res, v_res))
        del k, v
    return layers, n_comp, n_res


def layer_bytes(layer, k_res, v_res, n_res, batch, q_heads):
    """Algorithmic HBM bytes of one fused launch: streams (headers included) + block tables +
    scales/zeros + residual K/V + q + out."""
    n = layer.stream_bytes()
    n += 2 * batch * layer.kv_heads * n_res * 128 * k_res.element_size()
    n += 2 * batch * q_heads * 128 * 2
    return n


def run_ours(args, w, rank, world, device):
    from packkv_b200 import ops
    from packkv_b200 import parallel
    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    by_heads = args.shard == "heads" and world > 1
    layers, n_comp, n_res = build_layers(w, device, dtype, head_shard=(rank, world) if by_heads else None)
    B, Hq = w["batch"], w["q_heads"] // (world if by_heads else 1)
    gather_buf = torch.empty(world, B, Hq, 128, dtype=dtype, device=device) if by_heads else None
    g = torch.Generator(device=device).manual_seed(77 + rank)
    q_dev = [torch.randn(B, Hq, 128, generator=g, device=device, dtype=torch.float32).to(dtype) for _ in layers]
    out_dev = [torch.empty_like(q) for q in q_dev]
    flags = ops.new_flags(device)
    alg_bytes = sum(layer_bytes(L, kr, vr, n_res, B, Hq) for L, kr, vr in layers)

    def step_resident():
        for (L, kr, vr), q, o in zip(layers, q_dev, out_dev):
            ops.decode_attention(q, L, kr, vr, n_res, out=o, flags=flags)
            if by_heads:
                parallel.gather_heads(o, buffer=gather_buf)

    q_host = [q.cpu().pin_memory() for q in q_dev]
    out_host = [torch.empty(B, Hq, 128, dtype=dtype).pin_memory() for _ in layers]
    # End to end: every layer's q comes from pinned host memory and every layer's output goes back to
    # it.  The copies run on two side streams (double-buffered staging of q), so the upload of layer
    # l+1 and the download of layer l-1 overlap the kernel of layer l; all of them are inside the
    # timed region, which ends only after the last download.
    q_stage = [torch.empty(B, Hq, 128, dtype=dtype, device=device) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in layers]

    def upload(i):
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_free[i % 2])                  # the kernel that last read this staging buffer
            q_stage[i % 2].copy_(q_host[i], non_blocking=True)
            ev_in[i % 2].record(s_in)

    def step_e2e():
        main = torch.cuda.current_stream()
        for e in ev_free:
            e.record(main)
        upload(0)
        for i, ((L, kr, vr), oh, o) in enumerate(zip(layers, out_host, out_dev)):
            if i + 1 < len(layers):
                upload(i + 1)
            main.wait_event(ev_in[i % 2])
            ops.decode_attention(q_stage[i % 2], L, kr, vr, n_res, out=o, flags=flags)
            ev_free[i % 2].record(main)
            if by_heads:
                parallel.gather_heads(o, buffer=gather_buf)
            ev_done[i].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[i])
                oh.copy_(o, non_blocking=True)
        main.wait_stream(s_out)

    def timed(fn, steps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms], device=device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(args.warmup, 3)):
        step_resident()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    ms = timed(step_resident, args.steps)
    clocks = sampler.stop()
    if clocks["samples"] < 2:
        # the timed region was shorter than the sampling period: sample an untimed repeat of the same steps
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        t_end = time.perf_counter() + 0.8
        while time.perf_counter() < t_end:
            step_resident()
            torch.cuda.synchronize()
        clocks = sampler.stop()
        clocks["note"] = "sampled during an untimed repeat of the timed steps (the timed region was shorter than the sampling period)"
    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    torch.cuda.synchronize()
    if int(flags.item()) != 0:
        raise RuntimeError(f"device flags set: {int(flags.item())}")

    if rank != 0:
        return None
    ms_per_step = ms / args.steps
    tokens = B if by_heads else B * world
    peak, peak_kind = measured_peak_gbs()
    per_launch_ms = ms_per_step / len(layers)
    achieved = (alg_bytes / len(layers)) / (per_launch_ms * 1e-3) / 1e9
    line = {
        "metric": "fused decompress-attention decode throughput", "value": tokens / (ms_per_step * 1e-3), "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if by_heads else "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["name"], "layers": w["layers"], "batch_per_gpu": B, "context": w["ctx"],
                   "compressed_tokens": n_comp, "residual_tokens": n_res, "k_quant": w.get("k_mode", "channel"), "v_quant": "token",
                   "bits_k": w["bits_k"], "bits_v": w["bits_v"], "block": w["block"],
                   "l2": f"working set {alg_bytes / 1e9:.2f} GB per step and GPU >> 126 MB L2 (no flush needed)",
                   "sharding": "KV heads per rank + NCCL all-gather of outputs" if by_heads else "batch (independent sequences, no collective)"},
        "e2e": {"value": tokens / (ms_e2e / args.steps * 1e-3), "unit": "tok/s",
                "h2d_bytes_per_step": len(layers) * B * Hq * 128 * 2, "d2h_bytes_per_step": len(layers) * B * Hq * 128 * 2},
        "gpu_launches": len(layers) * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_kind,
                     "traffic": None if by_heads else NCU_TRAFFIC_BYTES.get(("attn", B, w["ctx"], w["kv_heads"], w["bits_k"], w["bits_v"], w["block"])),
                     "algorithmic_bytes_per_launch": alg_bytes // len(layers), "kernel": "attn_decode_kernel",
                     "avg_launch_ms": per_launch_ms},
        "compressed_kv_gbs": achieved,
        "clocks": clocks,
    }
    return line


# ------------------------------------------------------------------------------------------------
def cpu_reference_path(w, sample_batch: int, repeats: int, threads: int):
    """The reference's CPU path for one layer of `sample_batch` sequences: bit-unpack with its
    C++ codec (single-threaded by construction), dequantise and eager attention in torch."""
    import numpy as np
    from oracle import codec
    from oracle import quant as Q
    from packkv_b200 import synth
    torch.set_num_threads(threads)
    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    n_comp, n_res = split_context(w["ctx"], w["block"])
    k, v = synth.synth_kv(sample_batch, w["kv_heads"], w["ctx"], 128, seed=1000, dtype=dtype, apply_rope=True)
    q = synth.synth_q(sample_batch, w["q_heads"], 128, seed=1000, dtype=dtype)
    kc, kz, ks = Q.quant_ints(k[:, :, :n_comp], w["block"], synth.rel_for_bits(w["bits_k"]), "channel")
    vc, vz, vs = Q.quant_ints(v[:, :, :n_comp], w["block"], synth.rel_for_bits(w["bits_v"]), "token")
    refc = codec.reference()
    impl = refc if refc is not None and refc.supports("k", w["kv_heads"] * 128, w["cbk"], w["bits_k"]) else codec.restated()
    kind = "reference" if impl is refc else "port"
    vcb = 128 if kind == "reference" else w["cbv"]

    def seq_codes(c5, s):
        return c5[s].flatten(1, 2).permute(1, 0, 2).flatten(1, 2).contiguous().to(torch.uint8).numpy()

    packed = []
    for s in range(sample_batch):
        kk, vv = seq_codes(kc, s), seq_codes(vc, s)
        if vv.shape[0] % vcb:
            vv = np.concatenate([vv, np.zeros((vcb - vv.shape[0] % vcb, vv.shape[1]), np.uint8)])
        packed.append((impl.encode("k", kk, w["cbk"], w["bits_k"]), impl.encode("v", vv, vcb, w["bits_v"]), kk.shape, vv.shape))
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        kd_list, vd_list = [], []
        for (ke, ve, kshape, vshape) in packed:
            kcodes = impl.decode("k", ke[0], ke[1], kshape[0], kshape[1], w["cbk"], w["bits_k"])
            vcodes = impl.decode("v", ve[0], ve[1], vshape[0], vshape[1], vcb, w["bits_v"])[:n_comp]
            kd_list.append(torch.from_numpy(kcodes).view(n_comp, w["kv_heads"], 128).permute(1, 0, 2))
            vd_list.append(torch.from_numpy(vcodes).view(n_comp, w["kv_heads"], 128).permute(1, 0, 2))
        kq = torch.stack(kd_list).to(dtype).reshape(sample_batch, w["kv_heads"], -1, w["block"], 128)
        vq = torch.stack(vd_list).to(dtype).reshape(sample_batch, w["kv_heads"], -1, w["block"], 128)
        K = torch.cat([Q.dequant(kq, kz, ks), k[:, :, n_comp:]], 2)
        V = torch.cat([Q.dequant(vq, vz, vs), v[:, :, n_comp:]], 2)
        out = Q.eager_attention(q, K, V)
        times.append(time.perf_counter() - t0)
    times.sort()
    t_layer = times[len(times) // 2]
    tok_s = sample_batch / (t_layer * w["layers"])
    return tok_s, kind, t_layer, float(out.float().abs().max())


def run_reference(args, w):
    threads = os.cpu_count() or 1
    sample_batch = 2 if w["ctx"] <= 8192 else 1
    tok_s, kind, t_layer, _ = cpu_reference_path(w, sample_batch, repeats=max(5, min(args.steps, 100)), threads=threads)
    n_comp, n_res = split_context(w["ctx"], w["block"])
    sample = (f"1 layer x {sample_batch} sequences of the workload per step (median {t_layer * 1e3:.0f} ms): C++ bit-unpack "
              f"(1 thread) + torch dequantise + eager attention ({threads} threads); tok/s = sequences / (layer time x {w['layers']} layers)")
    return {
        "impl": "reference", "metric": "fused decompress-attention decode throughput", "value": tok_s, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_layer * w["layers"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["name"], "layers": w["layers"], "batch_per_gpu": w["batch"], "context": w["ctx"],
                   "compressed_tokens": n_comp, "residual_tokens": n_res, "k_quant": "channel", "v_quant": "token"},
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def run_encode(args, rank, world, device):
    """Encoder / append throughput on Mistral-7B-shaped KV: prefill-encode `batch` sequences of
    16384 tokens (K per-channel, V per-token, fp16), then append one token per step through the
    cache class.  Algorithmic bytes = fp16 K and V read + streams, block tables and parameters
    written.  Sequences are sharded over ranks (weak scaling, no collective)."""
    from packkv_b200 import cache as C
    from packkv_b200 import encode, synth
    from packkv_b200.config import PackKVCacheConfig, QuantMethod, QuantMode, RepackMethod
    B, H, S, bits, block = args.encode_batch, 8, 16384, args.encode_bits, args.encode_block
    dtype = torch.float16
    k, v = synth.synth_kv(B, H, S, 128, seed=3000 + rank, dtype=dtype, device=device, apply_rope=True)
    rel = synth.rel_for_bits(bits)
    kw = dict(block=block, bits_k=bits, bits_v=bits, k_rel=rel, v_rel=rel, k_mode=QuantMode.ChannelQuant)

    def timed(fn, steps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms], device=device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    layer = None
    for _ in range(max(args.warmup, 3)):
        layer = encode.compress_kv(k, v, **kw)
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    ms = timed(lambda: encode.compress_kv(k, v, **kw), args.steps) / args.steps
    clocks = sampler.stop()
    src_bytes = 2 * k.numel() * 2
    out_bytes = layer.stream_bytes()
    alg = src_bytes + out_bytes
    # append: 512 single-token steps on a cache prefilled with 1024 tokens
    C.PackKVCacheConfigStatic.config = PackKVCacheConfig("synthetic", QuantMethod.KIVI, RepackMethod.NONE, False, block, 128 + block, 16, rel, rel)
    cache = C.PackKVCache(B, H, 128, 1)
    cos, sin = synth.rope_tables(1024 + 512, 128, device=device, dtype=dtype)
    cache.update(k[:, :, :1024], v[:, :, :1024], 0, {"cos": cos[:, :1024], "sin": sin[:, :1024]})
    pos = [1024]

    def append_step():
        t = pos[0]
        cache.update(k[:, :, t:t + 1], v[:, :, t:t + 1], 0, {"cos": cos[:, t:t + 1], "sin": sin[:, t:t + 1]})
        pos[0] += 1
    ms_append = timed(append_step, 512) / 512
    cache._check_flags()
    C.PackKVCacheConfigStatic.config = None
    # end to end: K and V start in pinned host memory, the streams and their byte counts go back to it
    k_host, v_host = k.cpu().pin_memory(), v.cpu().pin_memory()
    ks_host = torch.empty(layer.k_stream.shape, dtype=torch.uint8).pin_memory()
    vs_host = torch.empty(layer.v_stream.shape, dtype=torch.uint8).pin_memory()
    nb_host = torch.empty(2, B, dtype=torch.int32).pin_memory()
    k_dev, v_dev = torch.empty_like(k), torch.empty_like(v)

    def step_e2e():
        k_dev.copy_(k_host, non_blocking=True)
        v_dev.copy_(v_host, non_blocking=True)
        L = encode.compress_kv(k_dev, v_dev, **kw)
        ks_host.copy_(L.k_stream, non_blocking=True)
        vs_host.copy_(L.v_stream, non_blocking=True)
        nb_host[0].copy_(L.k_bytes, non_blocking=True)
        nb_host[1].copy_(L.v_bytes, non_blocking=True)
    step_e2e()
    e2e_steps = max(1, min(args.steps, 5))
    ms_e2e = timed(step_e2e, e2e_steps) / e2e_steps
    if rank != 0:
        return None
    peak, peak_kind = measured_peak_gbs()
    achieved = alg / (ms * 1e-3) / 1e9
    return {
        "metric": "KV encode throughput", "value": world * alg / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"mistral-7b-shaped KV encode: {B} sequences x 16384 tokens x 8 KV heads x 128 per GPU, {bits}-bit, block {block}",
                   "l2": f"{alg / 1e9:.2f} GB per step >> 126 MB L2"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind,
                     "traffic": NCU_TRAFFIC_BYTES.get(("mistral7b-encode", B, bits, block)), "algorithmic_bytes_per_step": alg,
                     "kernel": "k/v_fused_encode_kernel + scan_sizes_kernel + compact_kernel (K and V): 6 launches per step"},
        "source_fp16_gbs": world * src_bytes / (ms * 1e-3) / 1e9,
        "compressed_over_fp16": out_bytes / src_bytes,
        "append": {"ms_per_token_step": ms_append, "sequences": B, "steps": 512,
                   "tokens_per_s": world * B / (ms_append * 1e-3)},
        "e2e": {"value": world * alg / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": src_bytes,
                "d2h_bytes_per_step": int(layer.k_stream.numel() + layer.v_stream.numel() + 8 * B)},
        "gpu_launches": 7 * args.steps, "clocks": clocks,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama8b", choices=sorted(WORKLOADS) + ["mistral7b-encode"])
    ap.add_argument("--encode-batch", type=int, default=16)
    ap.add_argument("--encode-bits", type=int, default=4)
    ap.add_argument("--encode-block", type=int, default=64)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--decode-bits-k", type=int, default=None, help="override the decode workload's K bit width (sweeps)")
    ap.add_argument("--decode-bits-v", type=int, default=None, help="override the decode workload's V bit width (sweeps)")
    ap.add_argument("--decode-k-mode", default="channel", choices=["channel", "token"], help="K quantisation parameters (sweeps)")
    ap.add_argument("--shard", default="batch", choices=["batch", "heads"],
                    help="multi-GPU split: independent sequences per rank (weak scaling, no collective) or KV heads per "
                         "rank with an all-gather of the outputs (strong scaling)")
    args = ap.parse_args()
    w = WORKLOADS.get(args.workload)
    if w is not None and (args.decode_bits_k or args.decode_bits_v or args.decode_k_mode != "channel"):
        w = dict(w, bits_k=args.decode_bits_k or w["bits_k"], bits_v=args.decode_bits_v or w["bits_v"], k_mode=args.decode_k_mode)
        w["name"] += f" [override: K {w['bits_k']}-bit {w['k_mode']}, V {w['bits_v']}-bit]"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if w is None:
            raise SystemExit("--impl reference is defined for the decode workloads")
        if rank == 0:
            print(json.dumps(run_reference(args, w)), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=device)
    if args.workload == "mistral7b-encode":
        line = run_encode(args, rank, world, device)
        if rank == 0:
            print(json.dumps(line), flush=True)
        if world > 1:
            torch.distributed.barrier()
            torch.distributed.destroy_process_group()
        return
    line = run_ours(args, w, rank, world, device)
    if rank == 0:
        if not args.no_cpu_baseline:
            t0 = time.perf_counter()
            nseq = 2 if w["ctx"] <= 8192 else 1
            reps = 120 if w["ctx"] <= 8192 else 30                     # ~10 s of CPU work: a stable median
            tok_s, kind, t_layer, _ = cpu_reference_path(w, nseq, repeats=reps, threads=os.cpu_count() or 1)
            line["cpu_baseline"] = {
                "value": tok_s, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": kind,
                "sample": f"1 layer x {nseq} sequences, median of {reps} runs ({t_layer * 1e3:.0f} ms each, {time.perf_counter() - t0:.0f} s in all "
                          f"with set-up): C++ bit-unpack (1 thread) + torch dequantise + eager attention (all threads); scaled by {w['layers']} layers"}
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
