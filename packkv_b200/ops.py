"""Device-tensor wrappers over the C ABI (include/packkv_sm100.h).

Everything here takes CUDA tensors, launches on torch's current stream and returns without
synchronising.  Tensors are only the carrier for device memory; the arithmetic is in
libpackkv_sm100.so.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import math

import torch

from . import _lib

HB = {"k": 128, "v": 64}


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("expected CUDA tensors; this library has no CPU path")


def k_block_bound(cb: int, bits: int) -> int:
    lb = 3 if bits >= 4 else 2
    r = cb // 16
    return 2 * r + r * (bits * 16 + lb * 16 + 128 * 2 * bits)


def v_block_bound(cb: int, bits: int) -> int:
    lb = 3 if bits >= 4 else 2
    rpw = 2 if cb == 128 else 1
    ppt = 2 if cb == 32 else 4
    nseg = 2 * rpw
    return 2 * nseg + nseg * (bits * ppt * 4 + lb * ppt * 4 + 32 * ppt * 2 * bits)


def block_bound(which: str, cb: int, bits: int) -> int:
    return k_block_bound(cb, bits) if which == "k" else v_block_bound(cb, bits)


def new_flags(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def encode_codes(which: str, codes: torch.Tensor, cb: int, bits: int, *, stream: Optional[torch.Tensor] = None,
                 info: Optional[torch.Tensor] = None, stream_bytes: Optional[torch.Tensor] = None,
                 flags: Optional[torch.Tensor] = None, first_cb: int = 0
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Bit-packs uint8 codes (n_seq, ctx, hidden) into per-sequence streams.

    Returns (stream (n_seq, capacity) u8, info (n_seq, n_blocks, 2) i32 holding u32 values,
    stream_bytes (n_seq,) i32, flags (1,) i32).  Passing the buffers of an earlier call with
    first_cb > 0 appends the new token blocks behind the existing ones.
    """
    _require_cuda(codes, stream, info, stream_bytes, flags)
    if codes.dtype != torch.uint8 or codes.dim() != 3 or not codes.is_contiguous():
        raise ValueError("codes must be a contiguous uint8 tensor (n_seq, ctx, hidden)")
    n_seq, ctx, hidden = codes.shape
    hb = HB[which]
    if cb <= 0 or ctx % cb or hidden % hb:
        raise ValueError("ctx must be a multiple of cb and hidden a multiple of the block width")
    nhid = hidden // hb
    nblk_new = (ctx // cb) * nhid
    dev = codes.device
    if info is None:
        info = torch.zeros(n_seq, first_cb * nhid + nblk_new, 2, dtype=torch.int32, device=dev)
    if stream is None:
        cap = (first_cb * nhid + nblk_new) * block_bound(which, cb, bits)
        stream = torch.zeros(n_seq, max(16, cap), dtype=torch.uint8, device=dev)
    if stream_bytes is None:
        stream_bytes = torch.zeros(n_seq, dtype=torch.int32, device=dev)
    if flags is None:
        flags = new_flags(dev)
    if info.shape[1] < first_cb * nhid + nblk_new:
        raise ValueError("block_info is too small for the appended blocks")
    fn = _lib.lib().pkv_k_encode if which == "k" else _lib.lib().pkv_v_encode
    st = fn(codes.data_ptr(), codes.stride(0), stream.data_ptr(), stream.stride(0), stream.shape[1],
            info.data_ptr(), info.shape[1], stream_bytes.data_ptr(), flags.data_ptr(),
            n_seq, ctx, hidden, cb, hb, bits, first_cb, _stream_ptr())
    _lib.check(st, f"{which}_encode")
    return stream, info, stream_bytes, flags


def decode_codes(which: str, stream: torch.Tensor, info: torch.Tensor, ctx: int, hidden: int, cb: int, bits: int, *,
                 valid_bytes: Optional[int] = None, flags: Optional[torch.Tensor] = None, first_cb: int = 0,
                 out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Unpacks per-sequence streams back to uint8 codes (n_seq, ctx, hidden)."""
    _require_cuda(stream, info, flags, out)
    if stream.dtype != torch.uint8 or stream.dim() != 2 or stream.stride(1) != 1:
        raise ValueError("stream must be a uint8 tensor (n_seq, capacity)")
    n_seq = stream.shape[0]
    hb = HB[which]
    if out is None:
        out = torch.zeros(n_seq, ctx, hidden, dtype=torch.uint8, device=stream.device)
    if flags is None:
        flags = new_flags(stream.device)
    fn = _lib.lib().pkv_k_decode if which == "k" else _lib.lib().pkv_v_decode
    st = fn(stream.data_ptr(), stream.stride(0), stream.shape[1] if valid_bytes is None else valid_bytes,
            info.data_ptr(), info.shape[1], out.data_ptr(), out.stride(0), flags.data_ptr(),
            n_seq, ctx, hidden, cb, hb, bits, first_cb, _stream_ptr())
    _lib.check(st, f"{which}_decode")
    return out, flags


K_CHANNEL, K_TOKEN, Q_VECTOR, Q_BLOCK = 0, 1, 2, 3


def _param_extents(scale: torch.Tensor, mode: int):
    """(capacity in blocks, capacity in tokens) of a parameter tensor of the given mode; the extent the mode does not
    use is 0."""
    if mode == K_CHANNEL:
        return scale.shape[2], 0
    if mode == K_TOKEN:
        return 0, scale.shape[1]
    if mode == Q_VECTOR:
        return 0, scale.shape[2]
    return scale.shape[1], 0


@dataclass
class Quantised:
    codes: torch.Tensor     # (B, S, H*128) uint8, the encoders' input layout
    scale: torch.Tensor     # channel: (B, H, capacity_blocks, 128); token: (B, capacity_tokens); vector: (B, H, capacity_tokens);
                            # block: (B, capacity_blocks)
    zero: torch.Tensor


def quantize(x: torch.Tensor, block: int, rel: float, mode, *, bits: int = 0, high_precision_zero: bool = False,
             flags: Optional[torch.Tensor] = None, capacity_tokens: Optional[int] = None,
             scale: Optional[torch.Tensor] = None, zero: Optional[torch.Tensor] = None, first_token: int = 0
             ) -> Quantised:
    """Block-quantises x (B, H, S, 128) fp16/bf16 like the reference's quant_ints.

    `mode` is a QuantMode or one of the integers K_CHANNEL / K_TOKEN / Q_VECTOR / Q_BLOCK (the last two are not
    taken by the encoder's single pass or the attention kernel: their codes go through encode_codes).
    Passing existing scale/zero tensors with first_token > 0 writes the new parameters behind
    the ones already there (append path).
    """
    _require_cuda(x, flags, scale, zero)
    if x.dim() != 4 or x.shape[3] != 128 or x.stride(3) != 1 or x.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("x must be (B, H, S, 128) fp16/bf16 with contiguous channels")
    m = getattr(mode, "value", mode)
    m = {"ChannelQuant": K_CHANNEL, "TokenQuant": K_TOKEN, "VectorQuant": Q_VECTOR, "BlockQuant": Q_BLOCK}.get(m, m)
    if m not in (K_CHANNEL, K_TOKEN, Q_VECTOR, Q_BLOCK):
        raise RuntimeError("not supported")
    B, H, S, D = x.shape
    if S % block:
        raise ValueError("Tensor shape is not divisible by block size")
    cap = max(S + first_token, capacity_tokens or 0)
    dev = x.device
    if flags is None:
        flags = new_flags(dev)
    codes = torch.empty(B, S, H * D, dtype=torch.uint8, device=dev)
    if scale is None:
        shape = {K_CHANNEL: (B, H, cap // block, D), K_TOKEN: (B, cap), Q_VECTOR: (B, H, cap), Q_BLOCK: (B, cap // block)}[m]
        scale = torch.zeros(shape, dtype=x.dtype, device=dev)
        zero = torch.zeros(shape, dtype=x.dtype, device=dev)
    pb, pt = _param_extents(scale, m)
    st = _lib.lib().pkv_quantize(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2), codes.data_ptr(), codes.stride(0),
                                 scale.data_ptr(), zero.data_ptr(), pb, first_token // block, pt, first_token,
                                 B, H, S, block, float(rel), bits, m, int(high_precision_zero),
                                 int(x.dtype == torch.bfloat16), flags.data_ptr(), _stream_ptr())
    _lib.check(st, "quantize")
    return Quantised(codes, scale, zero)


@dataclass
class CompressedLayer:
    """Device-resident compressed KV of one layer: per-sequence K and V streams with their
    block tables and quantisation parameters (layouts: include/packkv_sm100.h)."""
    k_stream: torch.Tensor      # (B, capacity) u8
    k_info: torch.Tensor        # (B, n_k_blocks, 2) i32 (u32 values)
    k_bytes: torch.Tensor       # (B,) i32
    k_scale: torch.Tensor       # channel: (B, Hkv, n_comp/cbk, 128); token: (B, n_comp)
    k_zero: torch.Tensor
    v_stream: torch.Tensor
    v_info: torch.Tensor
    v_bytes: torch.Tensor
    v_scale: torch.Tensor       # (B, n_comp)
    v_zero: torch.Tensor
    n_comp: int
    kv_heads: int
    cbk: int
    cbv: int
    bits_k: int
    bits_v: int
    k_mode: int
    high_precision_zero: bool = False
    order: Optional[torch.Tensor] = None   # (B, n_comp/block, block) u8 when tokens were reordered inside blocks

    def stream_bytes(self) -> int:
        """Compressed payload actually read by a decode step (streams + block tables + scales)."""
        n = int(self.k_bytes.sum().item()) + int(self.v_bytes.sum().item())
        n += self.k_info.numel() * 4 + self.v_info.numel() * 4
        for t in (self.k_scale, self.k_zero, self.v_scale, self.v_zero):
            n += t.numel() * t.element_size()
        return n


def _check_layer_shapes(L: "CompressedLayer", batch: int) -> None:
    """Host-side bounds of everything the attention kernel indexes from n_comp, kv_heads and the block sizes:
    a layer whose metadata disagrees with its arrays (a caller mistake, a truncated or corrupt blob) must raise
    here instead of reading outside the arrays on the device."""
    if L.cbk not in (64, 128) or L.cbv not in (64, 128) or L.n_comp <= 0 or L.kv_heads <= 0:
        raise RuntimeError("not supported") if L.cbk == 32 or L.cbv == 32 else ValueError("bad layer metadata")
    nkb, nvb = (L.n_comp // L.cbk) * L.kv_heads, (L.n_comp // L.cbv) * 2 * L.kv_heads
    for name in ("k_stream", "v_stream", "k_info", "v_info", "k_scale", "k_zero", "v_scale", "v_zero"):
        t = getattr(L, name)
        if t.shape[0] != batch:
            raise ValueError(f"{name} holds {t.shape[0]} sequences, q holds {batch}")
    if L.k_info.dim() != 3 or L.k_info.shape[2] != 2 or L.k_info.shape[1] < nkb or not L.k_info.is_contiguous():
        raise ValueError(f"k_info must be a contiguous (B, >= {nkb}, 2) table")
    if L.v_info.dim() != 3 or L.v_info.shape[2] != 2 or L.v_info.shape[1] < nvb or not L.v_info.is_contiguous():
        raise ValueError(f"v_info must be a contiguous (B, >= {nvb}, 2) table")
    if L.v_scale.dim() != 2 or L.v_scale.shape[1] < L.n_comp or L.v_zero.shape != L.v_scale.shape:
        raise ValueError("v_scale / v_zero must be (B, >= n_comp)")
    if L.k_mode == K_CHANNEL:
        want = (batch, L.kv_heads)
        if L.k_scale.dim() != 4 or tuple(L.k_scale.shape[:2]) != want or L.k_scale.shape[2] < L.n_comp // L.cbk or L.k_scale.shape[3] != 128 \
                or L.k_zero.shape != L.k_scale.shape:
            raise ValueError("channel-mode k_scale / k_zero must be (B, kv_heads, >= n_comp / cbk, 128)")
    elif L.k_scale.dim() != 2 or L.k_scale.shape[1] < L.n_comp or L.k_zero.shape != L.k_scale.shape:
        raise ValueError("token-mode k_scale / k_zero must be (B, >= n_comp)")
    if L.k_stream.dim() != 2 or L.v_stream.dim() != 2 or L.k_stream.stride(1) != 1 or L.v_stream.stride(1) != 1:
        raise ValueError("streams must be (B, capacity) with contiguous bytes")


# changes whenever the attention kernel changes in a way that can change its DRAM traffic (keys recorded profiler figures)
ATTN_KERNEL_REVISION = 3


def decode_attention(q: torch.Tensor, layer: Optional[CompressedLayer], k_res: Optional[torch.Tensor],
                     v_res: Optional[torch.Tensor], n_res: int, *, scaling: Optional[float] = None,
                     out: Optional[torch.Tensor] = None,
                     flags: Optional[torch.Tensor] = None, kv_heads: Optional[int] = None,
                     exchange: Optional["_lib.AttnExchange"] = None, append: Optional[tuple] = None,
                     scratch: Optional[torch.Tensor] = None, plan: Optional[tuple] = None, plan_only: bool = False):
    """softmax(q K^T * scaling) V for one query token per sequence.

    q: (B, Hq, 128) fp16/bf16 (post-RoPE).  `layer` holds the compressed tokens, k_res/v_res
    (B, Hkv, R_cap, 128) the uncompressed residual whose first n_res tokens are valid.
    Returns out (B, Hq, 128) in q's dtype; asynchronous on the current stream.  `exchange` (KV-head-sharded
    decode on several GPUs, see parallel.HeadExchange) makes the launch also deliver the rows to every rank.
    `append` = (k_new, v_new, cos, sin) with k_new / v_new (B, Hkv, 1, 128) and cos / sin (B or 1, 1, 128) or None:
    the launch writes the step's new token (K rotated like rope()) into residual row n_res - 1 before attending;
    n_res counts that token.
    `scratch` (new_attention_scratch) lets the library split a launch with few (sequence, KV head) pairs over
    several clusters per pair in two launches; `plan` = (cluster, nsplit, launches[, extra]), 0 = choose, forces the split
    (extra > 0 with cluster 1: the first `extra` pairs get nsplit + 1 CTAs).
    plan_only: nothing is launched and the plan (cluster, nsplit, launches, extra) that would be used is returned.
    """
    _require_cuda(q, k_res, v_res, out, flags, scratch)
    if q.dim() != 3 or q.shape[2] != 128 or not q.is_contiguous():
        raise ValueError("q must be a contiguous (B, Hq, 128) tensor")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("q must be fp16 or bf16")
    B, Hq, D = q.shape
    if layer is not None:
        kv_heads = layer.kv_heads
    elif kv_heads is None:
        kv_heads = k_res.shape[1]
    if Hq % kv_heads:
        raise ValueError("q heads must be a multiple of kv heads")
    if out is None:
        out = torch.empty_like(q)
    if flags is None:
        flags = new_flags(q.device)
    a = _lib.AttnArgs()
    a.q, a.out = q.data_ptr(), out.data_ptr()
    n_comp = 0 if layer is None else layer.n_comp
    if n_comp > 0:
        L = layer
        for t in (L.k_scale, L.k_zero, L.v_scale, L.v_zero):
            if t.dtype != q.dtype or not t.is_contiguous():
                raise ValueError("scale / zero tensors must be contiguous and of q's dtype")
        _check_layer_shapes(L, B)
        a.k_stream, a.k_seq_stride, a.k_capacity = L.k_stream.data_ptr(), L.k_stream.stride(0), L.k_stream.shape[1] & ~15
        a.k_info, a.k_info_seq_stride = L.k_info.data_ptr(), L.k_info.shape[1]
        a.k_scale, a.k_zero = L.k_scale.data_ptr(), L.k_zero.data_ptr()
        a.v_stream, a.v_seq_stride, a.v_capacity = L.v_stream.data_ptr(), L.v_stream.stride(0), L.v_stream.shape[1] & ~15
        a.v_info, a.v_info_seq_stride = L.v_info.data_ptr(), L.v_info.shape[1]
        a.v_scale, a.v_zero = L.v_scale.data_ptr(), L.v_zero.data_ptr()
        a.param_tokens = L.v_scale.shape[1]
        a.param_blocks = L.k_scale.shape[2] if L.k_mode == K_CHANNEL else 0
        if L.k_mode == K_TOKEN and L.k_scale.shape[1] != L.v_scale.shape[1]:
            raise ValueError("token-mode K and V parameter arrays must have the same row length")
        a.cbk, a.cbv, a.bits_k, a.bits_v = L.cbk, L.cbv, L.bits_k, L.bits_v
        a.k_mode, a.high_precision_zero = L.k_mode, int(L.high_precision_zero)
    if n_res > 0:
        if k_res.dtype != q.dtype or v_res.dtype != q.dtype or k_res.stride(3) != 1 or k_res.stride(2) != 128:
            raise ValueError("residual tensors must be (B, Hkv, R, 128) with contiguous rows, in q's dtype")
        if k_res.stride() != v_res.stride():
            raise ValueError("k_res and v_res must share strides")
        a.k_res, a.v_res = k_res.data_ptr(), v_res.data_ptr()
        a.res_seq_stride, a.res_head_stride = k_res.stride(0), k_res.stride(1)
    a.n_res, a.batch, a.kv_heads, a.group, a.n_comp = n_res, B, kv_heads, Hq // kv_heads, n_comp
    a.is_bf16 = int(q.dtype == torch.bfloat16)
    a.scaling = float(D ** -0.5 if scaling is None else scaling)
    a.flags = flags.data_ptr()
    if append is not None:
        k_new, v_new, cos, sin = append
        _require_cuda(k_new, v_new, cos, sin)
        if n_res < 1 or k_new.shape != (B, kv_heads, 1, 128) or v_new.shape != k_new.shape or k_new.stride(3) != 1 or v_new.stride(3) != 1 \
                or k_new.dtype != q.dtype or v_new.dtype != q.dtype:
            raise ValueError("append needs k_new / v_new of shape (B, Hkv, 1, 128) in q's dtype with contiguous channels")
        ap = _lib.AttnAppend()
        ap.new_k, ap.new_v = k_new.data_ptr(), v_new.data_ptr()
        ap.k_stride_b, ap.k_stride_h, ap.v_stride_b, ap.v_stride_h = k_new.stride(0), k_new.stride(1), v_new.stride(0), v_new.stride(1)
        if cos is not None:
            if cos.dtype != q.dtype or sin.dtype != q.dtype or cos.shape[-2:] != (1, 128) or sin.shape != cos.shape or not cos.is_contiguous() \
                    or not sin.is_contiguous():
                raise ValueError("cos / sin must be contiguous (B or 1, 1, 128) tensors of q's dtype")
            ap.cos, ap.sin, ap.cs_stride_b = cos.data_ptr(), sin.data_ptr(), (0 if cos.shape[0] == 1 else 128)
        ap.res_capacity = k_res.shape[2]
    else:
        ap = None
    if scratch is not None or plan is not None or plan_only:
        pl = _lib.AttnPlan()
        if plan is not None:
            pl.cluster, pl.nsplit, pl.launches = plan[:3]
            pl.extra = plan[3] if len(plan) > 3 else 0
        if scratch is not None and (scratch.dtype != torch.uint8 or not scratch.is_contiguous() or scratch.data_ptr() % 256):
            raise ValueError("scratch must be a contiguous uint8 tensor aligned to 256 bytes (new_attention_scratch)")
        sbytes = 0 if scratch is None else scratch.numel()
        if plan_only:
            _lib.check(_lib.lib().pkv_attention_plan(ctypes.byref(a), ctypes.byref(pl), sbytes, int(exchange is not None)), "attention_plan")
            return (pl.cluster, pl.nsplit, pl.launches, pl.extra)
        st = _lib.lib().pkv_decode_attention_split(ctypes.byref(a), ctypes.byref(ap) if ap is not None else None,
                                                   ctypes.byref(exchange) if exchange is not None else None, ctypes.byref(pl),
                                                   scratch.data_ptr() if scratch is not None else None, sbytes, _stream_ptr())
    elif ap is not None:
        st = _lib.lib().pkv_decode_attention_append(ctypes.byref(a), ctypes.byref(ap), ctypes.byref(exchange) if exchange is not None else None,
                                                    _stream_ptr())
    elif exchange is None:
        st = _lib.lib().pkv_decode_attention(ctypes.byref(a), _stream_ptr())
    else:
        st = _lib.lib().pkv_decode_attention_exchange(ctypes.byref(a), ctypes.byref(exchange), _stream_ptr())
    _lib.check(st, "decode_attention")
    return out


def new_attention_scratch(device, nbytes: int = 32 << 20) -> torch.Tensor:
    """Zeroed scratch for decode_attention's two-launch form (scores, per-CTA maxima and sums, per-cluster rows and
    arrival counters); launches that share one must be ordered on one stream."""
    return torch.zeros(nbytes, dtype=torch.uint8, device=device)


def exchange_wait(arrivals: torch.Tensor, n_ranks: int, expected: int, flags: torch.Tensor, max_polls: int = 2_000_000,
                  consume: bool = False) -> None:
    """Makes the current stream wait until this rank's n_ranks arrival counters have reached `expected`
    (modulo 2^32); after max_polls polls (a quarter of a microsecond apart) the wait gives up and sets FLAG_TIMEOUT.
    consume: `expected` is the arrivals of one step and is taken off the counters again once they are all there, so
    that the same call serves every step (CUDA graphs)."""
    _require_cuda(arrivals, flags)
    fn = _lib.lib().pkv_exchange_wait_consume if consume else _lib.lib().pkv_exchange_wait
    st = fn(arrivals.data_ptr(), n_ranks, expected & 0xFFFFFFFF, max_polls, flags.data_ptr(), _stream_ptr())
    _lib.check(st, "exchange_wait")


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(x * cos) + (rotate_half(x) * sin) with the reference's per-op rounding.
    x (B, H, T, D) with contiguous channels; cos/sin (B or 1, T, D)."""
    _require_cuda(x, cos, sin, out)
    if x.dim() != 4 or x.stride(3) != 1 or x.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("x must be (B, H, T, D) fp16/bf16 with contiguous channels")
    B, H, T, D = x.shape
    cos, sin = cos.to(x.dtype).contiguous(), sin.to(x.dtype).contiguous()
    if cos.shape[-2:] != (T, D) or sin.shape != cos.shape:
        raise ValueError("cos/sin must be (B or 1, T, D)")
    if out is None:
        out = torch.empty(B, H, T, D, dtype=x.dtype, device=x.device)
    cs_stride = 0 if cos.shape[0] == 1 else T * D
    st = _lib.lib().pkv_rope(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2), cos.data_ptr(), sin.data_ptr(), cs_stride,
                             out.data_ptr(), out.stride(0), out.stride(1), out.stride(2), B, H, T, D,
                             int(x.dtype == torch.bfloat16), _stream_ptr())
    _lib.check(st, "rope")
    return out


def append_residual(k_new: torch.Tensor, v_new: torch.Tensor, k_res: torch.Tensor, v_res: torch.Tensor, position: int,
                    cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None) -> None:
    """Writes the new tokens (B, H, T, 128) into rows [position, position+T) of the residual buffers
    (B, H, capacity, 128): K after RoPE (skipped when cos/sin are None), V as is.  One launch."""
    _require_cuda(k_new, v_new, k_res, v_res, cos, sin)
    B, H, T, D = k_new.shape
    if D != 128 or v_new.shape != k_new.shape or k_new.stride(3) != 1 or v_new.stride(3) != 1:
        raise ValueError("k_new and v_new must be (B, H, T, 128) with contiguous channels")
    if k_res.shape != v_res.shape or k_res.stride() != v_res.stride() or k_res.stride(3) != 1 or k_res.stride(2) != 128:
        raise ValueError("k_res and v_res must be (B, H, capacity, 128) with contiguous rows and equal strides")
    if k_res.dtype != k_new.dtype or v_new.dtype != k_new.dtype or k_new.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("dtype mismatch")
    cs_stride = 0
    if cos is not None:
        cos, sin = cos.to(k_new.dtype).contiguous(), sin.to(k_new.dtype).contiguous()
        if cos.shape[-2:] != (T, D) or sin.shape != cos.shape:
            raise ValueError("cos/sin must be (B or 1, T, 128)")
        cs_stride = 0 if cos.shape[0] == 1 else T * D
    st = _lib.lib().pkv_append_residual(
        k_new.data_ptr(), k_new.stride(0), k_new.stride(1), k_new.stride(2), v_new.data_ptr(), v_new.stride(0), v_new.stride(1), v_new.stride(2),
        cos.data_ptr() if cos is not None else None, sin.data_ptr() if sin is not None else None, cs_stride,
        k_res.data_ptr(), v_res.data_ptr(), k_res.stride(0), k_res.stride(1), k_res.shape[2], position, B, H, T,
        int(k_new.dtype == torch.bfloat16), _stream_ptr())
    _lib.check(st, "append_residual")


def dequantize(codes: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, heads: int, block: int, mode: int, *,
               first_token: int = 0, high_precision_zero: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """codes (B, T, heads*128) uint8 + scale/zero -> dense (B, heads, T, 128) in scale's dtype."""
    _require_cuda(codes, scale, zero, out)
    B, T, _ = codes.shape
    if out is None:
        out = torch.empty(B, heads, T, 128, dtype=scale.dtype, device=codes.device)
    pb, pt = _param_extents(scale, mode)
    st = _lib.lib().pkv_dequantize(codes.data_ptr(), codes.stride(0), scale.data_ptr(), zero.data_ptr(), pb, pt, first_token,
                                   out.data_ptr(), out.stride(0), out.stride(1), out.stride(2), B, heads, T, block, mode,
                                   int(high_precision_zero), int(scale.dtype == torch.bfloat16), _stream_ptr())
    _lib.check(st, "dequantize")
    return out


def _encode_args(which: str, x, block, rel, mode, bits, hp, cb, scale, zero, stream, info, stream_bytes, flags, first_token):
    B, H, S, D = x.shape
    a = _lib.EncodeArgs()
    a.x, a.stride_b, a.stride_h, a.stride_s = x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)
    a.scale, a.zero = scale.data_ptr(), zero.data_ptr()
    a.param_blocks = scale.shape[2] if mode == K_CHANNEL else 0
    a.param_tokens = scale.shape[1] if mode == K_TOKEN else 0
    a.stream, a.stream_seq_stride, a.capacity = stream.data_ptr(), stream.stride(0), stream.shape[1]
    a.block_info, a.info_seq_stride, a.stream_bytes = info.data_ptr(), info.shape[1], stream_bytes.data_ptr()
    a.flags = flags.data_ptr()
    a.batch, a.heads, a.tokens, a.first_token, a.qblock, a.cb = B, H, S, first_token, block, cb
    a.which = 0 if which == "k" else 1
    a.bits, a.mode, a.high_precision_zero, a.is_bf16, a.rel = bits, mode, int(hp), int(x.dtype == torch.bfloat16), float(rel)
    return a


def encode_tensor(which: str, x: torch.Tensor, block: int, rel: float, mode: int, bits: int, cb: int, *,
                  scale: torch.Tensor, zero: torch.Tensor, stream: torch.Tensor, info: torch.Tensor,
                  stream_bytes: torch.Tensor, flags: torch.Tensor, first_token: int = 0,
                  high_precision_zero: bool = False, scratch: Optional[torch.Tensor] = None,
                  order: Optional[torch.Tensor] = None, order_block: int = 64) -> None:
    """Quantises x (B, H, S, 128) and packs it behind the `first_token` tokens already in the
    streams (one C call).  `scratch` (uint8, >= B*S*H*128 bytes) holds the codes in between; one is
    allocated when not given.  `order` (B, S/order_block, order_block) uint8 (value_median_order): rows are read
    through it, i.e. the tokens of every reorder block are stored in that order (single-pass modes only:
    RuntimeError("not supported") otherwise)."""
    _require_cuda(x, scale, zero, stream, info, stream_bytes, flags, scratch)
    if x.dim() != 4 or x.shape[3] != 128 or x.stride(3) != 1 or x.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("x must be (B, H, S, 128) fp16/bf16 with contiguous channels")
    B, H, S, D = x.shape
    if S % block or S % cb:
        raise ValueError("Tensor shape is not divisible by block size")
    need = B * S * H * D
    if scratch is None:
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=x.device)
    a = _encode_args(which, x, block, rel, mode, bits, high_precision_zero, cb, scale, zero, stream, info, stream_bytes, flags, first_token)
    if order is not None:
        _require_cuda(order)
        if order.dtype != torch.uint8 or not order.is_contiguous() or order.numel() != B * S:
            raise ValueError("order must be a contiguous uint8 tensor with one entry per token")
        st = _lib.lib().pkv_encode_tensor_ordered(ctypes.byref(a), order.data_ptr(), order_block, scratch.data_ptr(), scratch.numel(), _stream_ptr())
    else:
        st = _lib.lib().pkv_encode_tensor(ctypes.byref(a), scratch.data_ptr(), scratch.numel(), _stream_ptr())
    _lib.check(st, f"encode_tensor({which})")


def value_median_order(v: torch.Tensor, block: int, rel: float, flags: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token order of every block by descending lower median of the V codes (stable on ties), computed from
    fp16/bf16 V (B, H <= 8, S, 128) without a code matrix: the same order as median_order on quantised codes.
    Returns (B, S/block, block) uint8."""
    _require_cuda(v, flags)
    if v.dim() != 4 or v.shape[3] != 128 or v.stride(3) != 1 or v.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("v must be (B, H, S, 128) fp16/bf16 with contiguous channels")
    B, H, S, _ = v.shape
    if S % block:
        raise ValueError("Tensor shape is not divisible by block size")
    order = torch.empty(B, S // block, block, dtype=torch.uint8, device=v.device)
    a = _lib.EncodeArgs()
    a.x, a.stride_b, a.stride_h, a.stride_s = v.data_ptr(), v.stride(0), v.stride(1), v.stride(2)
    a.batch, a.heads, a.tokens, a.which, a.mode = B, H, S, 1, K_TOKEN
    a.is_bf16, a.rel = int(v.dtype == torch.bfloat16), float(rel)
    a.flags = (flags if flags is not None else new_flags(v.device)).data_ptr()
    st = _lib.lib().pkv_value_median_order(ctypes.byref(a), order.data_ptr(), block, _stream_ptr())
    _lib.check(st, "value_median_order")
    return order


def encode_tensor_static(which: str, x: torch.Tensor, block: int, rel: float, mode: int, bits: int, cb: int, *,
                         scale: torch.Tensor, zero: torch.Tensor, stream: torch.Tensor, info: torch.Tensor,
                         stream_bytes: torch.Tensor, flags: torch.Tensor, first_token: int = 0,
                         high_precision_zero: bool = False) -> None:
    """encode_tensor for callers that must stay away from the device allocator (a serving engine's
    decode loop whose memory pool owns all free HBM: an allocation there can fail or stall the
    device).  The codes go through a 16 MiB array built into the library, so B*S*H*128 must not
    exceed that (ValueError otherwise), and calls must not overlap on the GPU because they share
    it.  The first call on a device resolves the array's address: make it before capturing streams.
    Results are identical to encode_tensor's."""
    _require_cuda(x, scale, zero, stream, info, stream_bytes, flags)
    if x.dim() != 4 or x.shape[3] != 128 or x.stride(3) != 1 or x.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("x must be (B, H, S, 128) fp16/bf16 with contiguous channels")
    if x.shape[2] % block or x.shape[2] % cb:
        raise ValueError("Tensor shape is not divisible by block size")
    a = _encode_args(which, x, block, rel, mode, bits, high_precision_zero, cb, scale, zero, stream, info, stream_bytes, flags, first_token)
    st = _lib.lib().pkv_encode_tensor_static(ctypes.byref(a), _stream_ptr())
    _lib.check(st, f"encode_tensor_static({which})")


def median_order(v_codes: torch.Tensor, heads: int, block: int, want_keys: bool = False):
    """Token order of every block by descending lower-median of the V codes (stable on ties).
    v_codes (B, S, heads*128) uint8 -> order (B, S/block, block) uint8 [, keys (B, S) uint8]."""
    _require_cuda(v_codes)
    B, S, _ = v_codes.shape
    order = torch.empty(B, S // block, block, dtype=torch.uint8, device=v_codes.device)
    keys = torch.empty(B, S, dtype=torch.uint8, device=v_codes.device) if want_keys else None
    st = _lib.lib().pkv_median_order(v_codes.data_ptr(), v_codes.stride(0), order.data_ptr(),
                                     keys.data_ptr() if want_keys else None, B, heads, S, block, _stream_ptr())
    _lib.check(st, "median_order")
    return (order, keys) if want_keys else order


def greedy_order(k_codes: torch.Tensor, v_codes: torch.Tensor, heads: int, block: int, pack_len: int = 16) -> torch.Tensor:
    """Token order of every block by the reference's greedy repacking heuristic
    (utils/compute.py:210-260) on the K||V code vectors of each token.
    k_codes, v_codes (B, S, heads*128) uint8 -> order (B, S/block, block) uint8."""
    _require_cuda(k_codes, v_codes)
    if k_codes.shape != v_codes.shape or k_codes.stride() != v_codes.stride():
        raise ValueError("k_codes and v_codes must have the same shape and strides")
    B, S, _ = k_codes.shape
    order = torch.empty(B, S // block, block, dtype=torch.uint8, device=k_codes.device)
    st = _lib.lib().pkv_greedy_order(k_codes.data_ptr(), v_codes.data_ptr(), k_codes.stride(0), order.data_ptr(),
                                     B, heads, S, block, pack_len, _stream_ptr())
    _lib.check(st, "greedy_order")
    return order


def size_model(codes: torch.Tensor, pack_len: int = 16) -> int:
    """Bytes the reference's bit_pack estimate (utils/compute.py:272-297) gives for one code tensor
    (B, S, hidden) uint8 (synchronises to read the two counters back)."""
    _require_cuda(codes)
    B, S, hidden = codes.shape
    bits = torch.zeros(1, dtype=torch.int64, device=codes.device)
    present = torch.zeros(8, dtype=torch.int32, device=codes.device)
    st = _lib.lib().pkv_size_model(codes.data_ptr(), codes.stride(0), B, S, hidden, pack_len, bits.data_ptr(), present.data_ptr(), _stream_ptr())
    _lib.check(st, "size_model")
    n_values = sum(bin(int(w) & 0xFFFFFFFF).count("1") for w in present.tolist())
    if n_values == 0:
        return 0
    b = math.ceil(math.log2(n_values))
    n_packs = B * (S // pack_len) * hidden
    return (int(bits.item()) * pack_len + n_packs * (b + math.ceil(math.log2(b + 1)))) // 8


def gather_rows(codes: torch.Tensor, order: torch.Tensor, block: int) -> torch.Tensor:
    """Applies `order` to the token rows of a code matrix (B, S, row_bytes)."""
    _require_cuda(codes, order)
    B, S, rb = codes.shape
    out = torch.empty_like(codes)
    st = _lib.lib().pkv_gather_rows(codes.data_ptr(), out.data_ptr(), codes.stride(0), order.data_ptr(), B, S, block, rb, _stream_ptr())
    _lib.check(st, "gather_rows")
    return out


def gather_params(params: torch.Tensor, order: torch.Tensor, block: int, tokens: int, first: int = 0) -> torch.Tensor:
    """Applies `order` to per-token parameters (B, row_len) for tokens [first, first+tokens)."""
    _require_cuda(params, order)
    out = params.clone()
    st = _lib.lib().pkv_gather_params(params.data_ptr(), out.data_ptr(), params.shape[1], first, order.data_ptr(),
                                      params.shape[0], tokens, block, _stream_ptr())
    _lib.check(st, "gather_params")
    return out
