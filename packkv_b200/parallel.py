"""Multi-GPU sharding of the decode path: one process per GPU, torch.distributed for plumbing.

Two ways to split the work, both without any exchange inside the kernels:

* batch sharding  - sequences are independent; rank r owns sequences [r*B/n, (r+1)*B/n).  No
  collective on the data path.
* KV-head sharding - rank r owns KV heads [r*H/n, (r+1)*H/n) and their q heads.  Streams are built
  from per-head blocks, so a rank packs only its heads.  Per-token quantisation parameters (V, and K
  in token mode) span ALL heads (reference QUANT_DIM, utils/compute.py:405-410), so the quantiser
  runs on the full tensor and only the rank's columns of the code matrix are packed; the parameters
  stay replicated.  The only collective is an all-gather of the attention outputs
  (batch x q_heads/n x 128 per rank and layer) over NCCL.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import ctypes

import torch
import torch.distributed as dist


def partition(n_items: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, even split; raises if it does not divide."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    if n_items % world:
        raise ValueError(f"{n_items} items do not divide over {world} ranks")
    per = n_items // world
    return rank * per, (rank + 1) * per


def q_heads_of(kv_lo: int, kv_hi: int, group: int) -> Tuple[int, int]:
    return kv_lo * group, kv_hi * group


def gather_heads(local_out: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                 buffer: Optional[torch.Tensor] = None) -> torch.Tensor:
    """all-gather of per-rank attention outputs (B, Hq/n, D) -> (B, Hq, D), rank-major heads."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    B, Hl, D = local_out.shape
    if buffer is None:
        buffer = torch.empty(world, B, Hl, D, dtype=local_out.dtype, device=local_out.device)
    dist.all_gather(list(buffer.unbind(0)), local_out.contiguous(), group=group)
    return buffer.permute(1, 0, 2, 3).reshape(B, world * Hl, D)


class _RawCuda:
    """Lets torch view device memory that this package allocated itself (uint8, 1-D)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


class HeadExchange:
    """Per-layer exchange of the KV-head-sharded attention outputs: every rank ends up with the rows of all
    ranks in a (world, B, Hq/world, 128) buffer, heads rank-major.

    mode "nccl": one all-gather per layer after the attention launch (the checked baseline).
    mode "peer": the attention launch itself stores its rows into every rank's buffer (buffers and arrival
    counters are shared between the processes of the node through CUDA IPC handles) and a one-warp kernel makes
    the stream wait for the other ranks' rows (and takes the step's arrivals off the counters again, so that a CUDA
    graph over the layer loop can be replayed); two buffers alternate, so a rank may run one step ahead of the
    slowest one.  Use: ``o = ops.decode_attention(..., exchange=x.begin()); x.gather(o)``.
    """

    def __init__(self, batch: int, q_heads_local: int, world: int, dtype, device, mode: str = "nccl",
                 group: Optional[dist.ProcessGroup] = None, rank: Optional[int] = None, kv_heads_local: Optional[int] = None,
                 flags: Optional[torch.Tensor] = None, max_polls: int = 2_000_000):
        if mode not in ("nccl", "peer"):
            raise ValueError(f"unknown exchange mode {mode!r}")
        self.mode, self.world, self.group = mode, world, group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.step, self.max_polls = 0, max_polls
        if mode == "nccl":
            self.buffer = torch.empty(world, batch, q_heads_local, 128, dtype=dtype, device=device)
            self._parts = list(self.buffer.unbind(0))
            return
        from . import _lib, ops
        if kv_heads_local is None:
            raise ValueError("peer mode needs kv_heads_local (arrivals per step = batch * kv_heads_local)")
        self.per_step = batch * kv_heads_local
        self.flags = ops.new_flags(device) if flags is None else flags
        slice_bytes = batch * q_heads_local * 128 * torch.empty((), dtype=dtype).element_size()
        buf_bytes = (world * slice_bytes + 255) // 256 * 256
        # one exportable allocation per rank: two gathered buffers, then two sets of arrival counters
        total = 2 * buf_bytes + 256
        ptr, hbuf = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        with torch.cuda.device(device):
            _lib.check(_lib.lib().pkv_exchange_alloc(total, ctypes.byref(ptr), hbuf), "exchange_alloc")
        self._own = ptr.value
        self._store = torch.as_tensor(_RawCuda(ptr.value, total), device=device)
        handles = [None] * world
        dist.all_gather_object(handles, (self.rank, hbuf.raw), group=group)
        self._mapped, base = [], [0] * world
        for r, h in handles:
            if r == self.rank:
                base[r] = self._own
            else:
                # mapped into THIS device's address space (the exporter's GPU becomes a peer of this one)
                mp_ = ctypes.c_void_p()
                with torch.cuda.device(device):
                    _lib.check(_lib.lib().pkv_ipc_open(ctypes.c_char_p(h), ctypes.byref(mp_)), "ipc_open")
                self._mapped.append(mp_.value)
                base[r] = mp_.value
        self.buffers = [self._store[i * buf_bytes:i * buf_bytes + world * slice_bytes].view(dtype).view(world, batch, q_heads_local, 128)
                        for i in range(2)]
        self._arrivals = [self._store[2 * buf_bytes + 128 * i:2 * buf_bytes + 128 * i + 4 * world].view(torch.int32) for i in range(2)]
        self._x = []
        for i in range(2):
            x = _lib.AttnExchange()
            x.n_ranks, x.rank = world, self.rank
            for r in range(world):
                x.gathered[r] = base[r] + i * buf_bytes
                x.arrivals[r] = base[r] + 2 * buf_bytes + 128 * i
            self._x.append(x)
        self.buffer = self.buffers[0]
        dist.barrier(group=group)

    def close(self):
        """Unmaps the other ranks' buffers (after all ranks have stopped using the exchange)."""
        from . import _lib
        for p in getattr(self, "_mapped", []):
            _lib.lib().pkv_ipc_close(p)
        self._mapped = []
        if getattr(self, "_own", None):
            torch.cuda.synchronize()
            self.buffers = self._arrivals = self._store = self.buffer = None
            _lib.lib().pkv_exchange_free(self._own)
            self._own = None

    def begin(self):
        """The exchange block for the next attention launch (peer mode; None in nccl mode)."""
        return None if self.mode == "nccl" else self._x[self.step & 1]

    def gather(self, local_out: torch.Tensor) -> torch.Tensor:
        if self.mode == "nccl":
            dist.all_gather(self._parts, local_out, group=self.group)
            return self.buffer
        from . import ops
        i = self.step & 1
        self.step += 1
        # consuming wait: the same launch every step, so the layer loop can live in a CUDA graph
        ops.exchange_wait(self._arrivals[i], self.world, self.per_step, self.flags, self.max_polls, consume=True)
        self.buffer = self.buffers[i]
        return self.buffer

    def full(self) -> torch.Tensor:
        """(B, Hq, 128) copy of the last gathered result."""
        w, B, Hl, D = self.buffer.shape
        return self.buffer.permute(1, 0, 2, 3).reshape(B, w * Hl, D)


def check_against_full(w: dict, rank: int, world: int, device, dtype, shard_layer0, q_full0: torch.Tensor, n_comp: int, n_res: int,
                       xchg: "HeadExchange", flags: torch.Tensor, scratch: Optional[torch.Tensor] = None, plan=None) -> dict:
    """Runs layer 0 of a head-sharded benchmark workload once more: every rank computes its heads and takes part
    in the exchange; rank 0 also computes all heads on its own GPU from the same seeded K/V, with the same CTAs per
    (sequence, KV head) as the sharded launch (the order of the fp32 sums depends on nothing else), and compares."""
    from . import encode, ops, synth
    from .config import QuantMode
    layer, k_res, v_res = shard_layer0
    Hq_l = q_full0.shape[1] // world
    q_l = q_full0[:, rank * Hq_l:(rank + 1) * Hq_l].contiguous()
    x = xchg.begin()
    used = ops.decode_attention(q_l, layer, k_res, v_res, n_res, flags=flags, scratch=scratch, plan=plan, plan_only=True, exchange=x)
    out = ops.decode_attention(q_l, layer, k_res, v_res, n_res, flags=flags, exchange=x, scratch=scratch, plan=plan)
    xchg.gather(out)
    torch.cuda.synchronize()
    got = xchg.full()
    if rank != 0:
        return {}
    k, v = synth.synth_kv(w["batch"], w["kv_heads"], w["ctx"], 128, seed=1000, dtype=dtype, device=device, apply_rope=True)
    full = encode.compress_kv(k[:, :, :n_comp], v[:, :, :n_comp], block=w["block"], bits_k=w["bits_k"], bits_v=w["bits_v"],
                              k_rel=synth.rel_for_bits(w["bits_k"]), v_rel=synth.rel_for_bits(w["bits_v"]),
                              k_mode=QuantMode.TokenQuant if w.get("k_mode") == "token" else QuantMode.ChannelQuant, cbk=w["cbk"], cbv=w["cbv"])
    big = ops.new_attention_scratch(device, 256 << 20) if used[2] == 2 else None
    ref = ops.decode_attention(q_full0, full, k[:, :, n_comp:].contiguous(), v[:, :, n_comp:].contiguous(), n_res, flags=flags, scratch=big, plan=used)
    torch.cuda.synchronize()
    return {"bit_identical_to_one_gpu": bool(torch.equal(got, ref)), "max_abs_diff": float((got.float() - ref.float()).abs().max()),
            "plan": {"cluster": used[0], "clusters_per_pair": used[1], "launches": used[2], "pairs_with_one_more_cta": used[3]}}


def compress_kv_head_shard(k: torch.Tensor, v: torch.Tensor, rank: int, world: int, *, block: int, bits_k: int, bits_v: int,
                           k_rel: float, v_rel: float, k_mode, cbk: Optional[int] = None, cbv: Optional[int] = None):
    """Builds the rank's compressed layer from the FULL K, V (B, Hkv, S, 128): quantise with
    all-head statistics, pack only this rank's heads.  Returns (layer, (kv_lo, kv_hi))."""
    from . import encode, ops
    from .config import QuantMode
    B, H, S, D = k.shape
    lo, hi = partition(H, rank, world)
    Hs = hi - lo
    cbk = block if cbk is None else cbk
    cbv = block if cbv is None else cbv
    km = ops.K_CHANNEL if k_mode == QuantMode.ChannelQuant else ops.K_TOKEN
    flags = ops.new_flags(k.device)
    kq = ops.quantize(k, block, k_rel, km, bits=bits_k, flags=flags)
    vq = ops.quantize(v, block, v_rel, ops.K_TOKEN, bits=bits_v, flags=flags)
    kc = kq.codes.view(B, S, H, D)[:, :, lo:hi].reshape(B, S, Hs * D).contiguous()
    vc = vq.codes.view(B, S, H, D)[:, :, lo:hi].reshape(B, S, Hs * D).contiguous()
    k_stream = torch.zeros(B, encode.stream_capacity("k", S, Hs, cbk, bits_k), dtype=torch.uint8, device=k.device)
    v_stream = torch.zeros(B, encode.stream_capacity("v", S, Hs, cbv, bits_v), dtype=torch.uint8, device=k.device)
    _, k_info, k_bytes, _ = ops.encode_codes("k", kc, cbk, bits_k, stream=k_stream, flags=flags)
    _, v_info, v_bytes, _ = ops.encode_codes("v", vc, cbv, bits_v, stream=v_stream, flags=flags)
    k_scale = kq.scale[:, lo:hi].contiguous() if km == ops.K_CHANNEL else kq.scale
    k_zero = kq.zero[:, lo:hi].contiguous() if km == ops.K_CHANNEL else kq.zero
    layer = ops.CompressedLayer(k_stream=k_stream, k_info=k_info, k_bytes=k_bytes, k_scale=k_scale, k_zero=k_zero,
                                v_stream=v_stream, v_info=v_info, v_bytes=v_bytes, v_scale=vq.scale, v_zero=vq.zero,
                                n_comp=S, kv_heads=Hs, cbk=cbk, cbv=cbv, bits_k=bits_k, bits_v=bits_v, k_mode=km)
    return layer, (lo, hi)


def max_over_ranks(ms: float, device) -> float:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
