"""Headline benchmark: fused decompress-attention decode over a compressed KV cache.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload llama8b]

Workload (default): Llama-3.1-8B-shaped decode attention -- 32 layers, 32 q heads / 8 KV heads,
head_dim 128, bf16, batch 16, context 8192 (8064 compressed tokens + 128 uncompressed residual
tokens per the cache's cut rule), K per-channel 4 bit in 64-token blocks, V per-token 4 bit packed
in 128-token blocks: the stream layouts the reference's codec writes and reads.  Synthetic KV
(packkv_b200.synth) stands in for real-model caches.  One STEP = one decode step's attention for
all layers = 32 launches of the fused kernel producing `batch` tokens.

Multi-GPU (torchrun, one rank per GPU): sequences are independent, so the batch is sharded with
no data-path collective; every rank holds a full `batch` of sequences (weak scaling) and the
reported value is (all ranks' tokens) / (max over ranks of the device time).

JSON line: metric decode tok/s; `value` with q/out resident in HBM; `e2e` through the public
API with q in pinned host memory and the output read back every layer; `roofline` on the
algorithmic compressed bytes of the fused kernel; `cpu_baseline` (one GPU only) = the reference's
own CPU path (C++ bit-unpack + torch dequantise + eager attention) on a bounded sample.  The
default workload's line also carries the other parts of the metric as extra keys:
`v_block_64` (the same decode with 64-token V blocks), `encode` (Mistral-7B-shaped KV encode, 64
sequences x 16384 tokens split over the ranks, with and without the median reorder, and the
single-token append), `phi3_e2e` (Phi-3-mini-shaped model generating 256 tokens after a 4096-token
prompt, 8 sequences per GPU) and, on more than one GPU, `head_sharded` (the long-context workload split
by KV heads with the output exchange).
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
                    block=64, cbk=64, cbv=128, name="llama-3.1-8b-shaped decode attention, batch 16, ctx 8192, 4-bit K/V, block 64"),
    "qwen8b-long": dict(layers=36, batch=8, q_heads=32, kv_heads=8, ctx=32768, dtype="bf16", bits_k=2, bits_v=4,
                        block=128, cbk=128, cbv=128, name="qwen3-8b-shaped decode attention, batch 8, ctx 32768, 2-bit K / 4-bit V, block 128"),
    "llama8b-2l": dict(layers=2, batch=16, q_heads=32, kv_heads=8, ctx=8192, dtype="bf16", bits_k=4, bits_v=4,
                       block=64, cbk=64, cbv=128, name="2 layers of the llama-3.1-8b-shaped workload (profiling case)"),
    "tiny": dict(layers=2, batch=2, q_heads=8, kv_heads=2, ctx=1024, dtype="bf16", bits_k=4, bits_v=4,
                 block=64, cbk=64, cbv=64, name="tiny smoke workload"),
}
RECENT = 192   # buffer_size of every reference script (128 + 64)
MIN_TIMED_S = 1.0   # the timed region is repeated until it is at least this long

# dram__bytes_read.sum + dram__bytes_write.sum of one launch (attention) or one step (encoder) from the ncu
# captures kept with the repository's profile summaries.  An entry is valid for one revision of the kernel only (the revision is
# a constant of packkv_b200.ops that changes with the kernel): other revisions report null.
NCU_TRAFFIC_BYTES = {
    ("attn", 3, 16, 8192, 8, 4, 4, 64, 128): 160.9e6,      # 155.96 MB read + 4.92 MB written
    ("encode", 2, 16, 4, 64): 1401e6,                      # K 576 + 151 MB, V 561 + 113 MB
    ("encode", 2, 64, 4, 64): 4 * 1401e6,                  # the 16-sequence capture scaled by the sequences (traffic is per sequence)
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


def timed_batches(fn, steps: int, world: int, device, min_seconds: float = MIN_TIMED_S, max_batches: int = 400):
    """Times batches of `steps` calls of fn with CUDA events on the current stream (barrier and synchronize on
    both sides of every batch, max over ranks) until the batches add up to min_seconds.  Returns
    (median batch ms, number of batches, total ms)."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    batches = []
    while len(batches) < max_batches:
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
        batches.append(ms)
        if sum(batches) >= min_seconds * 1e3:       # the same decision on every rank: ms is the max over ranks
            break
    s = sorted(batches)
    return s[len(s) // 2], len(batches), sum(batches)


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
        # the V token block may exceed the quantisation block: only whole V blocks are compressed
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


def time_decode(w, steps, warmup, rank, world, device, *, by_heads=False, with_e2e=True, sample_clocks=True, exchange="nccl", graph=False):
    """Builds the workload's compressed layers on this rank and times decode steps.  Returns a dict of raw
    measurements (milliseconds are per step, max over ranks)."""
    from packkv_b200 import ops, parallel
    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    by_heads = by_heads and world > 1
    layers, n_comp, n_res = build_layers(w, device, dtype, head_shard=(rank, world) if by_heads else None)
    B, Hq = w["batch"], w["q_heads"] // (world if by_heads else 1)
    g = torch.Generator(device=device).manual_seed(77 + (0 if by_heads else rank))
    q_full = [torch.randn(B, w["q_heads"] if by_heads else Hq, 128, generator=g, device=device, dtype=torch.float32).to(dtype) for _ in layers]
    q_dev = [q[:, rank * Hq:(rank + 1) * Hq].contiguous() if by_heads else q for q in q_full]
    out_dev = [torch.empty_like(q) for q in q_dev]
    flags = ops.new_flags(device)
    alg_bytes = sum(layer_bytes(L, kr, vr, n_res, B, Hq) for L, kr, vr in layers)
    xchg = parallel.HeadExchange(B, Hq, world, dtype, device, mode=exchange, rank=rank, kv_heads_local=w["kv_heads"] // world,
                                 flags=flags) if by_heads else None
    # scratch of the two-launch form (several clusters per (sequence, KV head)): the library uses it when the
    # launch has too few pairs to fill the GPU; w["plan"] forces (cluster, nsplit, launches)
    scratch = ops.new_attention_scratch(device, 64 << 20) if w.get("split", True) else None
    plan = w.get("plan")
    L0, kr0, vr0 = layers[0]
    used = ops.decode_attention(q_dev[0], L0, kr0, vr0, n_res, flags=flags, scratch=scratch, plan=plan, plan_only=True,
                                exchange=xchg.begin() if by_heads and xchg.mode == "peer" else None)

    def step_resident():
        for (L, kr, vr), q, o in zip(layers, q_dev, out_dev):
            ops.decode_attention(q, L, kr, vr, n_res, out=o, flags=flags, exchange=xchg.begin() if by_heads else None, scratch=scratch, plan=plan)
            if by_heads:
                xchg.gather(o)

    res = {"n_comp": n_comp, "n_res": n_res, "layers": len(layers), "batch": B, "q_heads_local": Hq, "alg_bytes": alg_bytes,
           "plan": {"cluster": used[0], "clusters_per_pair": used[1], "launches": used[2], "pairs_with_one_more_cta": used[3]}}
    for _ in range(max(warmup, 3)):
        step_resident()
    step_eager = step_resident
    graph = graph and len(layers) % 2 == 0 and (not by_heads or exchange == "peer")   # the exchange's two buffers alternate per layer
    if graph:
        # the whole layer loop (attention launches, exchange blocks, waits) as one CUDA graph: no host work per launch
        torch.cuda.synchronize()
        cuda_graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(cuda_graph, stream=side):
                step_eager()
        torch.cuda.current_stream().wait_stream(side)
        step_resident = cuda_graph.replay
        for _ in range(3):
            step_resident()
    res["cuda_graph"] = bool(graph)
    sampler = None
    if sample_clocks:
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
    ms, nb, total = timed_batches(step_resident, steps, world, device)
    if sampler is not None:
        res["clocks"] = sampler.stop()
        res["clocks"]["timed_region_s"] = round(total / 1e3, 3)
    res.update(ms_per_step=ms / steps, batches=nb, launches=len(layers) * steps * nb)

    if by_heads:
        # the kernels alone (every rank its own heads, nothing exchanged): the difference is what the exchange costs
        def step_local():
            for (L, kr, vr), q, o in zip(layers, q_dev, out_dev):
                ops.decode_attention(q, L, kr, vr, n_res, out=o, flags=flags, scratch=scratch, plan=plan)
        if graph:
            torch.cuda.synchronize()
            g_local = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(g_local, stream=side):
                    step_local()
            torch.cuda.current_stream().wait_stream(side)
            step_local = g_local.replay
        ms_l, _, _ = timed_batches(step_local, steps, world, device, min_seconds=0.3)
        res["exchange_ms_per_step"] = max(0.0, ms / steps - ms_l / steps)
        res["check"] = parallel.check_against_full(w, rank, world, device, dtype, layers[0], q_full[0], n_comp, n_res, xchg, flags, scratch=scratch,
                                                      plan=plan)

    if with_e2e:
        # End to end: every layer's q comes from pinned host memory and every layer's output goes back to
        # it.  The copies run on two side streams (double-buffered staging of q), so the upload of layer
        # l+1 and the download of layer l-1 overlap the kernel of layer l; all of them are inside the
        # timed region, which ends only after the last download.
        q_host = [q.cpu().pin_memory() for q in q_dev]
        out_host = [torch.empty(B, Hq, 128, dtype=dtype).pin_memory() for _ in layers]
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
                ops.decode_attention(q_stage[i % 2], L, kr, vr, n_res, out=o, flags=flags, exchange=xchg.begin() if by_heads else None, scratch=scratch, plan=plan)
                ev_free[i % 2].record(main)
                if by_heads:
                    xchg.gather(o)
                ev_done[i].record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[i])
                    oh.copy_(o, non_blocking=True)
            main.wait_stream(s_out)

        for _ in range(2):
            step_e2e()
        ms_e, _, _ = timed_batches(step_e2e, steps, world, device)
        res["ms_per_step_e2e"] = ms_e / steps
    torch.cuda.synchronize()
    if int(flags.item()) != 0:
        raise RuntimeError(f"device flags set: {int(flags.item())}")
    return res


def decode_line(args, w, rank, world, device):
    from packkv_b200 import ops
    m = time_decode(w, args.steps, args.warmup, rank, world, device, by_heads=args.shard == "heads", with_e2e=True)
    if rank != 0:
        return None
    by_heads = args.shard == "heads" and world > 1
    B, L = m["batch"], m["layers"]
    tokens = B if by_heads else B * world
    peak, peak_kind = measured_peak_gbs()
    per_launch_ms = m["ms_per_step"] / L
    achieved = (m["alg_bytes"] / L) / (per_launch_ms * 1e-3) / 1e9
    traffic = None if by_heads else NCU_TRAFFIC_BYTES.get(
        ("attn", ops.ATTN_KERNEL_REVISION, B, w["ctx"], w["kv_heads"], w["bits_k"], w["bits_v"], w["cbk"], w["cbv"]))
    line = {
        "metric": "fused decompress-attention decode throughput", "value": tokens / (m["ms_per_step"] * 1e-3), "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": m["ms_per_step"],
        "higher_is_better": True, "scaling": "strong" if by_heads else "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["name"], "layers": L, "batch_per_gpu": B, "context": w["ctx"],
                   "compressed_tokens": m["n_comp"], "residual_tokens": m["n_res"], "k_quant": w.get("k_mode", "channel"), "v_quant": "token",
                   "bits_k": w["bits_k"], "bits_v": w["bits_v"], "block": w["block"],
                   "stream_layout": f"K blocks of {w['cbk']} tokens x 128 channels, V blocks of {w['cbv']} tokens x 64 channels"
                                    + (" (the reference codec's V layout)" if w["cbv"] == 128 else " (no reference bitstream for this V layout)"),
                   "timed_batches": m["batches"],
                   "l2": f"working set {m['alg_bytes'] / 1e9:.2f} GB per step and GPU >> 126 MB L2 (no flush needed)",
                   "sharding": "KV heads per rank + exchange of outputs" if by_heads else "batch (independent sequences, no collective)"},
        "e2e": {"value": tokens / (m["ms_per_step_e2e"] * 1e-3), "unit": "tok/s",
                "h2d_bytes_per_step": L * B * m["q_heads_local"] * 128 * 2, "d2h_bytes_per_step": L * B * m["q_heads_local"] * 128 * 2},
        "gpu_launches": m["launches"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_kind, "traffic": traffic,
                     "algorithmic_bytes_per_launch": m["alg_bytes"] // L, "kernel": "attn_decode_kernel",
                     "avg_launch_ms": per_launch_ms},
        "compressed_kv_gbs": achieved,
        "clocks": m["clocks"],
    }
    return line


# ------------------------------------------------------------------------------------------------
def cpu_reference_path(w, sample_batch: int, repeats: int, threads: int):
    """The reference's CPU path for one layer of `sample_batch` sequences: bit-unpack with its
    C++ codec (single-threaded by construction), dequantise and eager attention in torch.
    Returns (codec kind, list of seconds per run)."""
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
        Q.eager_attention(q, K, V)
        times.append(time.perf_counter() - t0)
    return kind, times


def run_reference(args, w):
    """The reference arm: one STEP = the reference's CPU path over ALL sequences of ONE layer of the workload
    (that is what ms_per_step times); the decode rate of the whole model is that time times the layer count."""
    threads = os.cpu_count() or 1
    seqs = w["batch"]
    kind, times = cpu_reference_path(w, seqs, repeats=max(1, args.warmup) + args.steps, threads=threads)
    times = sorted(times[max(1, args.warmup):])
    t_layer = times[len(times) // 2]
    tok_s = seqs / (t_layer * w["layers"])
    n_comp, n_res = split_context(w["ctx"], w["block"])
    sample = (f"one step = 1 layer x all {seqs} sequences of the workload (median {t_layer * 1e3:.0f} ms over {len(times)} steps): C++ bit-unpack "
              f"(1 thread) + torch dequantise + eager attention ({threads} threads); tok/s = sequences / (step time x {w['layers']} layers)")
    return {
        "impl": "reference", "metric": "fused decompress-attention decode throughput", "value": tok_s, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_layer * 1e3,
        "step_is": "one layer of the workload", "layers_per_token": w["layers"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["name"], "layers": w["layers"], "batch_per_gpu": w["batch"], "context": w["ctx"],
                   "compressed_tokens": n_comp, "residual_tokens": n_res, "k_quant": "channel", "v_quant": "token"},
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ------------------------------------------------------------------------------------------------
def encode_leg(steps, warmup, rank, world, device, *, total_seqs=64, bits=4, block=64, with_median=True, with_e2e=True, with_append=True):
    """Encoder / append throughput on Mistral-7B-shaped KV (8 KV heads x 128, fp16): prefill-encode `total_seqs`
    sequences of 16384 tokens split evenly over the ranks (K per-channel, V per-token), without and with the
    median token reorder, then append one token per step for 512 steps through the cache class.  Algorithmic
    bytes = fp16 K and V read + streams, block tables and parameters written.  No collective: the value is
    (all ranks' bytes) / (max over ranks of the device time)."""
    from packkv_b200 import cache as C
    from packkv_b200 import encode, synth
    from packkv_b200.config import PackKVCacheConfig, QuantMethod, QuantMode, RepackMethod
    B, H, S = max(1, total_seqs // world), 8, 16384
    dtype = torch.float16
    k, v = synth.synth_kv(B, H, S, 128, seed=3000 + rank, dtype=dtype, device=device, apply_rope=True)
    rel = synth.rel_for_bits(bits)
    kw = dict(block=block, bits_k=bits, bits_v=bits, k_rel=rel, v_rel=rel, k_mode=QuantMode.ChannelQuant)
    peak, peak_kind = measured_peak_gbs()
    src_bytes = 2 * k.numel() * 2
    out = {"config": {"workload": f"mistral-7b-shaped KV encode: {B * world} sequences x 16384 tokens x 8 KV heads x 128 over {world} GPU(s), "
                                  f"fp16, {bits}-bit, block {block}", "sequences_per_gpu": B,
                      "l2": f"{2 * src_bytes / 1e9:.2f} GB per step and GPU >> 126 MB L2"}}
    for name, method in (("plain", RepackMethod.NONE), ("median", RepackMethod.MEDIAN)):
        if method == RepackMethod.MEDIAN and not with_median:
            continue
        layer = None
        for _ in range(max(warmup, 3)):
            layer = encode.compress_kv(k, v, repack_method=method, **kw)
        ms, nb, _ = timed_batches(lambda: encode.compress_kv(k, v, repack_method=method, **kw), max(1, min(steps, 10)), world, device, min_seconds=0.5)
        ms /= max(1, min(steps, 10))
        out_bytes = layer.stream_bytes() + (0 if layer.order is None else layer.order.numel())
        alg = src_bytes + out_bytes
        achieved = alg / (ms * 1e-3) / 1e9
        out[name] = {"value": world * achieved, "unit": "GB/s", "ms_per_step": ms, "source_fp16_gbs": world * src_bytes / (ms * 1e-3) / 1e9,
                     "compressed_over_fp16": out_bytes / src_bytes,
                     "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                                  "peak_source": peak_kind, "algorithmic_bytes_per_step": alg,
                                  "traffic": NCU_TRAFFIC_BYTES.get(("encode", ENCODE_REVISION, B, bits, block)) if method == RepackMethod.NONE else None}}
        del layer
    if with_append:
        # append: 512 single-token decode steps on a cache prefilled with 1024 tokens.  (a) update() + attend(): the
        # attention launch writes the new token itself, every 64th step a block is compressed; (b) attend() alone on
        # the same cache; the difference is what appending costs per token step.  (c) update() alone: the
        # separate append launch that a caller without the fused attention pays.
        C.PackKVCacheConfigStatic.config = PackKVCacheConfig("synthetic", QuantMethod.KIVI, RepackMethod.NONE, False, block, 128 + block, 16, rel, rel)
        cos, sin = synth.rope_tables(1024 + 1100, 128, device=device, dtype=dtype)
        q = synth.synth_q(B, 4 * H, 128, seed=9, dtype=dtype, device=device)

        def fresh():
            c = C.PackKVCache(B, 4 * H, 128, 1)
            c.update(k[:, :, :1024], v[:, :, :1024], 0, {"cos": cos[:, :1024], "sin": sin[:, :1024]})
            return c, [1024]
        cache, pos = fresh()

        def step_update():
            t = pos[0]
            cache.update(k[:, :, t:t + 1], v[:, :, t:t + 1], 0, {"cos": cos[:, t:t + 1], "sin": sin[:, t:t + 1]})
            pos[0] += 1

        def step_both():
            step_update()
            cache.attend(q, 0)
        for _ in range(3):
            step_both()
        ms_both, _, _ = timed_batches(step_both, 512, world, device, min_seconds=0.0, max_batches=1)
        cache.check_flags()
        # attention alone at the middle length of those steps
        cache = C.PackKVCache(B, 4 * H, 128, 1)
        cache.update(k[:, :, :1024 + 256], v[:, :, :1024 + 256], 0, {"cos": cos[:, :1280], "sin": sin[:, :1280]})
        for _ in range(3):
            cache.attend(q, 0)
        ms_attend, _, _ = timed_batches(lambda: cache.attend(q, 0), 512, world, device, min_seconds=0.0, max_batches=1)
        cache.check_flags()
        cache, pos = fresh()
        for _ in range(3):
            step_update()
        ms_update, _, _ = timed_batches(step_update, 512, world, device, min_seconds=0.0, max_batches=1)
        cache.check_flags()
        C.PackKVCacheConfigStatic.config = None
        out["append"] = {"us_per_token_step": max(0.0, ms_both - ms_attend) / 512 * 1e3, "update_plus_attend_us": ms_both / 512 * 1e3,
                         "attend_only_us": ms_attend / 512 * 1e3, "separate_append_launch_us": ms_update / 512 * 1e3,
                         "sequences_per_gpu": B, "steps": 512, "token_appends_per_s": world * B / (max(1e-6, ms_both - ms_attend) / 512 * 1e-3)}
    if with_e2e:
        # End to end: K and V start in pinned host memory, the streams and their byte counts go back to it.  The
        # sequences go through in groups on three streams (upload, encode, download), so that the uploads of one group
        # overlap the encode and the downloads of the groups before it; the timed region ends after the last download.
        layer = encode.compress_kv(k, v, **kw)
        groups = 4 if B % 4 == 0 and B >= 8 else 1
        G = B // groups
        k_host, v_host = k.cpu().pin_memory(), v.cpu().pin_memory()
        ks_host = torch.empty(layer.k_stream.shape, dtype=torch.uint8).pin_memory()
        vs_host = torch.empty(layer.v_stream.shape, dtype=torch.uint8).pin_memory()
        nb_host = torch.empty(2, B, dtype=torch.int32).pin_memory()
        k_dev, v_dev = torch.empty_like(k), torch.empty_like(v)
        s_in, s_out, s_cmp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        ev_in = [torch.cuda.Event() for _ in range(groups)]
        ev_cmp = [torch.cuda.Event() for _ in range(groups)]

        def step_e2e():
            s_in.wait_stream(s_cmp)                               # the device buffers of the step before are free again
            kept = []
            for g in range(groups):
                sl = slice(g * G, (g + 1) * G)
                with torch.cuda.stream(s_in):
                    k_dev[sl].copy_(k_host[sl], non_blocking=True)
                    v_dev[sl].copy_(v_host[sl], non_blocking=True)
                    ev_in[g].record(s_in)
                s_cmp.wait_event(ev_in[g])
                L = encode.compress_kv(k_dev[sl], v_dev[sl], **kw)
                ev_cmp[g].record(s_cmp)
                kept.append(L)                                    # its buffers stay alive until the downloads have run
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[g])
                    ks_host[sl].copy_(L.k_stream, non_blocking=True)
                    vs_host[sl].copy_(L.v_stream, non_blocking=True)
                    nb_host[0, sl].copy_(L.k_bytes, non_blocking=True)
                    nb_host[1, sl].copy_(L.v_bytes, non_blocking=True)
            s_cmp.wait_stream(s_out)
            return kept
        step_e2e()
        torch.cuda.synchronize()
        ms_e2e, _, _ = timed_batches(step_e2e, 2, world, device, min_seconds=0.0, max_batches=1)
        ms_e2e /= 2
        alg = src_bytes + layer.stream_bytes()
        out["e2e"] = {"value": world * alg / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": src_bytes,
                      "d2h_bytes_per_step": int(layer.k_stream.numel() + layer.v_stream.numel() + 8 * B), "sequence_groups": groups}
    return out if rank == 0 else None


def phi3_e2e_leg(rank, world, device, *, seqs_per_gpu=8, prompt=4096, new_tokens=256, layers=32):
    """Phi-3-mini-shaped end-to-end decode (32 layers, 32 heads without grouping, head_dim 96, hidden 3072, bf16,
    random-initialised weights, random prompt ids): prefill of `prompt` tokens, then `new_tokens` greedy steps of
    the unmodified transformers model whose decode attention runs on the compressed cache through the
    registered attention function.  Every GPU serves `seqs_per_gpu` sequences (batch sharding, no collective);
    value = generated tokens of all ranks / max over ranks of the decode-loop device time."""
    from transformers import Phi3Config, Phi3ForCausalLM
    from packkv_b200 import hf
    from packkv_b200.cache import PackKVCacheConfigStatic
    from packkv_b200.config import PackKVCacheConfig, QuantMethod, RepackMethod
    torch.manual_seed(1234)
    cfg = Phi3Config(hidden_size=3072, num_attention_heads=32, num_key_value_heads=32, num_hidden_layers=layers, intermediate_size=8192,
                     vocab_size=32064, max_position_embeddings=prompt + new_tokens + 64, pad_token_id=0, bos_token_id=1, eos_token_id=2)
    with torch.device(device):
        model = Phi3ForCausalLM(cfg).to(torch.bfloat16).eval()
    hf.register()
    model.set_attn_implementation(hf.ATTN_NAME)
    PackKVCacheConfigStatic.config = PackKVCacheConfig("phi-3-mini-shaped", QuantMethod.KIVI, RepackMethod.NONE, False, 64, 192, 16, 1 / 14, 1 / 14)
    try:
        g = torch.Generator(device=device).manual_seed(99 + rank)
        ids = torch.randint(3, 32000, (seqs_per_gpu, prompt), generator=g, device=device)
        cache = hf.make_cache(cfg, seqs_per_gpu)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        with torch.no_grad():
            ev[0].record()
            nxt = model(ids, past_key_values=cache, use_cache=True, logits_to_keep=1).logits[:, -1].argmax(-1, keepdim=True)
            if world > 1:
                torch.distributed.barrier()
            torch.cuda.synchronize()
            ev[1].record()
            for _ in range(new_tokens):
                nxt = model(nxt, past_key_values=cache, use_cache=True).logits[:, -1].argmax(-1, keepdim=True)
            ev[2].record()
            torch.cuda.synchronize()
        cache.check_flags()
        ms_prefill, ms_decode = ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])
        # the attention launches alone, on the final cache (one token more or less does not matter)
        q = torch.randn(seqs_per_gpu, 32, 1, 96, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
        for _ in range(2):
            for li in range(layers):
                cache.attend(q, li)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(8):
            for li in range(layers):
                cache.attend(q, li)
        a1.record()
        torch.cuda.synchronize()
        ms_attn_step = a0.elapsed_time(a1) / 8
        if world > 1:
            t = torch.tensor([ms_decode, ms_prefill], device=device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms_decode, ms_prefill = float(t[0]), float(t[1])
        kv_tokens = cache.get_seq_length(0)
        comp = cache.compressed_bytes()
        return {"workload": f"phi-3-mini-shaped model, {layers} layers, 32 heads x 96, bf16, random weights: {seqs_per_gpu} sequences per GPU x "
                            f"{world} GPU(s), prompt {prompt}, {new_tokens} generated tokens, 4-bit K (per channel) / V (per token), block 64",
                "value": world * seqs_per_gpu * new_tokens / (ms_decode * 1e-3), "unit": "tok/s", "ms_per_token_step": ms_decode / new_tokens,
                "prefill_ms": ms_prefill, "attention_ms_per_token_step": ms_attn_step, "attention_share": ms_attn_step / (ms_decode / new_tokens),
                "kv_tokens_at_end": kv_tokens, "compressed_stream_bytes_per_gpu": comp,
                "fp_kv_bytes_per_gpu": 2 * layers * seqs_per_gpu * 32 * kv_tokens * 96 * 2,
                "layout_note": "head_dim 96 is stored in 128-channel blocks (the tail repeats 32 channels): no reference bitstream exists for it"}
    finally:
        PackKVCacheConfigStatic.config = None
        del model
        torch.cuda.empty_cache()


ENCODE_REVISION = 2   # changes when the encoder kernels change (keys NCU_TRAFFIC_BYTES)


def legacy_matvec_leg(device, *, ctx=65536, hidden=1024, bits=4, layers=32, repeats=20):
    """The reference's two-kernel API on its own benchmark shape (scripts/throughput_config_test.py: hidden 1024,
    one sequence, context 64 K, 4 bit; it reports the sum over 32 layers of the wv kernel's time): K blocks of 64
    tokens x 128 channels through kq_mat_vec_mul, V blocks of 128 tokens x 64 channels through wv_mat_vec_mul,
    each timed by the call itself (CUDA events inside the call, like the reference's), median of `repeats`."""
    import packkv_cuda
    from packkv_b200 import ops, synth
    heads, dtype = hidden // 128, torch.float16
    k, v = synth.synth_kv(1, heads, ctx, 128, seed=3, dtype=dtype, device=device, apply_rope=True)
    out = {"shape": f"hidden {hidden}, context {ctx}, 1 sequence, {bits} bit", "layers": layers}
    for name, x, cb, hb in (("kq", k, 64, 128), ("wv", v, 128, 64)):
        flags = ops.new_flags(device)
        qz = ops.quantize(x, 64, synth.rel_for_bits(bits), ops.K_TOKEN, bits=bits, flags=flags)
        stream, info, nbytes, _ = ops.encode_codes("k" if name == "kq" else "v", qz.codes, cb, bits)
        stream = stream[0, : (int(nbytes[0].item()) + 15) // 16 * 16].contiguous()
        vec = torch.randn(heads, 128 if name == "kq" else ctx, dtype=dtype, device=device)
        res = torch.zeros(heads, ctx, dtype=dtype, device=device) if name == "kq" else torch.zeros(heads, 128, dtype=torch.float32, device=device)
        fn = packkv_cuda.kq_mat_vec_mul if name == "kq" else packkv_cuda.wv_mat_vec_mul
        times = sorted(fn(stream, info[0].contiguous(), vec, res, ctx, hidden, cb, hb, bits) for _ in range(repeats + 3))
        ms = times[len(times) // 2]
        out[name] = {"ms_per_call": ms, "ms_sum_over_layers": ms * layers, "stream_gbs": stream.numel() / (ms * 1e-3) / 1e9}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama8b", choices=sorted(WORKLOADS) + ["mistral7b-encode", "phi3-e2e", "legacy-matvec"])
    ap.add_argument("--encode-batch", type=int, default=64, help="sequences in all (split over the ranks)")
    ap.add_argument("--encode-bits", type=int, default=4)
    ap.add_argument("--encode-block", type=int, default=64)
    ap.add_argument("--encode-plain-only", action="store_true", help="encode workload: skip the median / append / end-to-end legs (sweeps)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="default workload: skip the v_block_64 / low_batch / long_context / encode / phi3_e2e / head_sharded legs")
    ap.add_argument("--decode-bits-k", type=int, default=None, help="override the decode workload's K bit width (sweeps)")
    ap.add_argument("--decode-bits-v", type=int, default=None, help="override the decode workload's V bit width (sweeps)")
    ap.add_argument("--decode-cbv", type=int, default=None, choices=[64, 128], help="override the V token block (sweeps)")
    ap.add_argument("--decode-batch", type=int, default=None, help="override the batch (sweeps)")
    ap.add_argument("--decode-ctx", type=int, default=None, help="override the context length (sweeps)")
    ap.add_argument("--decode-layers", type=int, default=None, help="override the number of layers (sweeps, profiling)")
    ap.add_argument("--decode-k-mode", default="channel", choices=["channel", "token"], help="K quantisation parameters (sweeps)")
    ap.add_argument("--shard", default="batch", choices=["batch", "heads"],
                    help="multi-GPU split: independent sequences per rank (weak scaling, no collective) or KV heads per "
                         "rank with an exchange of the outputs (strong scaling)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="output exchange of --shard heads")
    args = ap.parse_args()
    w = WORKLOADS.get(args.workload)
    overridden = w is not None and (args.decode_bits_k or args.decode_bits_v or args.decode_k_mode != "channel" or args.decode_cbv
                                    or args.decode_batch or args.decode_ctx or args.decode_layers)
    if overridden:
        w = dict(w, bits_k=args.decode_bits_k or w["bits_k"], bits_v=args.decode_bits_v or w["bits_v"], k_mode=args.decode_k_mode,
                 cbv=args.decode_cbv or w["cbv"], batch=args.decode_batch or w["batch"], ctx=args.decode_ctx or w["ctx"], layers=args.decode_layers or w["layers"])
        w["name"] += f" [override: batch {w['batch']}, ctx {w['ctx']}, K {w['bits_k']}-bit {w['k_mode']}, V {w['bits_v']}-bit, V block {w['cbv']}]"
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
    try:
        if args.workload == "mistral7b-encode":
            rest = not args.encode_plain_only
            leg = encode_leg(args.steps, args.warmup, rank, world, device, total_seqs=args.encode_batch, bits=args.encode_bits,
                             block=args.encode_block, with_median=rest, with_e2e=rest, with_append=rest)
            if rank == 0:
                p = leg["plain"]
                line = {"metric": "KV encode throughput", "value": p["value"], "unit": "GB/s", "n_gpus": world, "steps": args.steps,
                        "warmup": max(args.warmup, 3), "ms_per_step": p["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": leg["config"], "roofline": p["roofline"],
                        "e2e": leg.get("e2e"), "median_reorder": leg.get("median"), "append": leg.get("append"),
                        "source_fp16_gbs": p["source_fp16_gbs"], "compressed_over_fp16": p["compressed_over_fp16"], "gpu_launches": 2 * args.steps}
                print(json.dumps(line), flush=True)
            return
        if args.workload == "legacy-matvec":
            if rank == 0:
                leg = legacy_matvec_leg(device)
                print(json.dumps({"metric": "legacy two-kernel API, wv_mat_vec_mul summed over 32 layers", "value": leg["wv"]["ms_sum_over_layers"],
                                  "unit": "ms", "n_gpus": 1, "higher_is_better": False, "data": "synthetic", "detail": leg}), flush=True)
            return
        if args.workload == "phi3-e2e":
            leg = phi3_e2e_leg(rank, world, device)
            if rank == 0:
                print(json.dumps({"metric": "end-to-end decode throughput with the compressed KV cache", "value": leg["value"], "unit": "tok/s",
                                  "n_gpus": world, "steps": 256, "warmup": 0, "ms_per_step": leg["ms_per_token_step"], "higher_is_better": True,
                                  "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": {"workload": leg["workload"]},
                                  "detail": leg}), flush=True)
            return
        line = decode_line(args, w, rank, world, device)
        extras = args.workload == "llama8b" and not overridden and not args.no_extras and args.shard == "batch"
        if extras:
            torch.cuda.empty_cache()
            # the same decode with 64-token V blocks (this library's own layout; 8 layers are enough for a per-layer time)
            w64 = dict(w, cbv=64, layers=8)
            m = time_decode(w64, args.steps, args.warmup, rank, world, device, with_e2e=False, sample_clocks=False)
            if rank == 0:
                peak, _ = measured_peak_gbs()
                us = m["ms_per_step"] / m["layers"] * 1e3
                gbs = m["alg_bytes"] / m["layers"] / (us * 1e-6) / 1e9
                line["v_block_64"] = {"us_per_layer": us, "tok_s_at_32_layers": w["batch"] * world / (us * 1e-6 * 32), "compressed_kv_gbs": gbs,
                                      "roofline_frac": gbs / peak, "layers_timed": m["layers"]}
            torch.cuda.empty_cache()
            # one sequence at long contexts (the regime of the reference's own throughput scripts): few (sequence, KV
            # head) pairs, so the library splits each pair over several clusters in two launches; beside it the
            # single launch (one cluster of at most 16 CTAs per pair)
            low = {}
            for ctx in (32768, 131072):
                wl = dict(w, batch=1, ctx=ctx, layers=4)
                ms_ = time_decode(wl, args.steps, args.warmup, rank, world, device, with_e2e=False, sample_clocks=False)
                mo_ = time_decode(dict(wl, split=False), args.steps, args.warmup, rank, world, device, with_e2e=False, sample_clocks=False)
                if rank == 0:
                    peak, _ = measured_peak_gbs()
                    us = ms_["ms_per_step"] / ms_["layers"] * 1e3
                    gbs = ms_["alg_bytes"] / ms_["layers"] / (us * 1e-6) / 1e9
                    low[f"batch1_ctx{ctx}"] = {"us_per_layer": us, "tok_s_at_32_layers": world / (us * 1e-6 * 32), "compressed_kv_gbs": gbs,
                                               "roofline_frac": gbs / peak, "plan": ms_["plan"],
                                               "single_launch_us_per_layer": mo_["ms_per_step"] / mo_["layers"] * 1e3, "layers_timed": ms_["layers"]}
                torch.cuda.empty_cache()
            if rank == 0:
                line["low_batch"] = low
            if world == 1:
                # the long-context configuration on one GPU (at several GPUs the head_sharded leg below measures it)
                wq = dict(WORKLOADS["qwen8b-long"], layers=6)
                mq = time_decode(wq, max(5, args.steps // 2), args.warmup, rank, world, device, with_e2e=False, sample_clocks=False)
                peak, _ = measured_peak_gbs()
                us = mq["ms_per_step"] / mq["layers"] * 1e3
                gbs = mq["alg_bytes"] / mq["layers"] / (us * 1e-6) / 1e9
                line["long_context"] = {"workload": wq["name"], "layers_timed": mq["layers"], "us_per_layer": us,
                                        "tok_s_at_36_layers": wq["batch"] / (us * 1e-6 * 36), "compressed_kv_gbs": gbs, "roofline_frac": gbs / peak,
                                        "plan": mq["plan"]}
                torch.cuda.empty_cache()
            # a leg that fails must not take the line with it: its key then holds the error
            try:
                leg = encode_leg(args.steps, args.warmup, rank, world, device)
            except Exception as e:                      # noqa: BLE001
                leg = {"error": repr(e)[:300]}
            if rank == 0:
                line["encode"] = leg
            torch.cuda.empty_cache()
            try:
                leg = phi3_e2e_leg(rank, world, device)
            except Exception as e:                      # noqa: BLE001
                leg = {"error": repr(e)[:300]}
            if rank == 0:
                line["phi3_e2e"] = leg
            torch.cuda.empty_cache()
            if world > 1:
                try:
                    wq = dict(WORKLOADS["qwen8b-long"], layers=6)
                    mh = time_decode(wq, max(5, args.steps), args.warmup, rank, world, device, by_heads=True, with_e2e=False, sample_clocks=False,
                                     exchange=args.exchange, graph=True)
                    m1 = time_decode(wq, max(5, args.steps), args.warmup, rank, 1, device, with_e2e=False, sample_clocks=False, graph=True) if rank == 0 else None
                    torch.distributed.barrier()
                    if rank == 0:
                        us_n = mh["ms_per_step"] / mh["layers"] * 1e3
                        us_1 = m1["ms_per_step"] / m1["layers"] * 1e3
                        line["head_sharded"] = {
                            "workload": wq["name"], "layers_timed": mh["layers"], "exchange": args.exchange, "cuda_graph": mh["cuda_graph"],
                            "tok_s_at_36_layers": wq["batch"] / (us_n * 1e-6 * 36), "us_per_layer": us_n,
                            "exchange_us_per_layer": mh["exchange_ms_per_step"] / mh["layers"] * 1e3,
                            "one_gpu_us_per_layer": us_1, "speedup": us_1 / us_n, "efficiency": us_1 / us_n / world, "check": mh["check"]}
                except Exception as e:                # noqa: BLE001
                    if rank == 0:
                        line["head_sharded"] = {"error": repr(e)[:300]}
        if rank == 0:
            if not args.no_cpu_baseline and world == 1:
                t0 = time.perf_counter()
                nseq = 2 if w["ctx"] <= 8192 else 1
                reps = 60 if w["ctx"] <= 8192 else 15                      # a few seconds of CPU work: a stable median
                kind, times = cpu_reference_path(w, nseq, repeats=reps, threads=os.cpu_count() or 1)
                t_layer = sorted(times)[len(times) // 2]
                line["cpu_baseline"] = {
                    "value": nseq / (t_layer * w["layers"]), "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": kind,
                    "sample": f"1 layer x {nseq} sequences, median of {reps} runs ({t_layer * 1e3:.0f} ms each, {time.perf_counter() - t0:.0f} s in all "
                              f"with set-up): C++ bit-unpack (1 thread) + torch dequantise + eager attention (all threads); scaled by {w['layers']} layers"}
            print(json.dumps(line), flush=True)
    finally:
        if world > 1:
            torch.distributed.barrier()
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
