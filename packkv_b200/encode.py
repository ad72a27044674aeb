"""KV encoder front end: fp16/bf16 K and V -> device-resident compressed layer.

quantise (per-channel or per-token K, per-token V)  ->  optional in-block token reorder  ->
bit-pack into per-sequence streams.  All arithmetic runs in libpackkv_sm100.so.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .config import QuantMode, RepackMethod


def _pad16(n: int) -> int:
    return (n + 15) // 16 * 16


def stream_capacity(which: str, n_tokens: int, kv_heads: int, cb: int, bits: int) -> int:
    """Worst-case bytes of one sequence's stream for n_tokens tokens (16-byte multiple)."""
    nhid = kv_heads * (128 // ops.HB[which])
    return _pad16((n_tokens // cb) * nhid * ops.block_bound(which, cb, bits)) + 16


def compress_kv(k: torch.Tensor, v: torch.Tensor, *, block: int, bits_k: int, bits_v: int,
                k_rel: float, v_rel: float, k_mode: QuantMode = QuantMode.ChannelQuant,
                cbk: Optional[int] = None, cbv: Optional[int] = None, high_precision_zero: bool = False,
                capacity_tokens: Optional[int] = None, flags: Optional[torch.Tensor] = None,
                repack_method: RepackMethod = RepackMethod.NONE) -> ops.CompressedLayer:
    """Compresses K, V of shape (B, Hkv, S, 128) (S a multiple of the block sizes).

    `capacity_tokens` reserves stream and table room for later appends.  With
    RepackMethod.MEDIAN the tokens of every quantisation block are reordered (same order for K and
    V) by the descending median of their V codes before packing, with RepackMethod.GREEDY by the
    reference's greedy pack-building heuristic on the K||V codes; both narrow the per-pack value
    ranges, attention over the block is unaffected and `order` is kept for dense reconstruction.
    """
    if k.shape != v.shape or k.dim() != 4 or k.shape[3] != 128:
        raise ValueError("k and v must both be (B, Hkv, S, 128)")
    B, H, S, D = k.shape
    cbk = block if cbk is None else cbk
    cbv = block if cbv is None else cbv
    cap_tok = max(S, capacity_tokens or 0)
    dev = k.device
    # one cleared allocation for everything that must start at zero: the two byte counters and the flag word
    zeros = torch.zeros(2 * B + 1, dtype=torch.int32, device=dev)
    if flags is None:
        flags = zeros[2 * B:]
    km = ops.K_CHANNEL if k_mode == QuantMode.ChannelQuant else ops.K_TOKEN
    if k_mode not in (QuantMode.ChannelQuant, QuantMode.TokenQuant):
        raise RuntimeError("not supported")
    k_shape = (B, H, cap_tok // block, D) if km == ops.K_CHANNEL else (B, cap_tok)
    # parameters and block tables are written by the encoder for every token / block that is ever read: no clearing
    k_scale, k_zero = torch.empty(k_shape, dtype=k.dtype, device=dev), torch.empty(k_shape, dtype=k.dtype, device=dev)
    v_scale, v_zero = torch.empty(B, cap_tok, dtype=k.dtype, device=dev), torch.empty(B, cap_tok, dtype=k.dtype, device=dev)
    # streams need no clearing: every byte that is ever read has been written by an encoder
    k_stream = torch.empty(B, stream_capacity("k", cap_tok, H, cbk, bits_k), dtype=torch.uint8, device=dev)
    v_stream = torch.empty(B, stream_capacity("v", cap_tok, H, cbv, bits_v), dtype=torch.uint8, device=dev)
    k_info = torch.empty(B, (cap_tok // cbk) * H, 2, dtype=torch.int32, device=dev)
    v_info = torch.empty(B, (cap_tok // cbv) * 2 * H, 2, dtype=torch.int32, device=dev)
    k_bytes, v_bytes = zeros[:B], zeros[B:2 * B]
    fused_median = (repack_method == RepackMethod.MEDIAN and not high_precision_zero and block == 64 and H <= 8 and cbv % 64 == 0
                    and (cbk == block if km == ops.K_CHANNEL else cbk % 64 == 0)
                    and k.stride(3) == 1 and v.stride(3) == 1 and all(t.stride(i) % 8 == 0 for t in (k, v) for i in range(3)))
    if fused_median:
        # the order straight from V, then the single-pass encoder reads K and V rows through it: no code matrix in HBM
        order = ops.value_median_order(v, block, v_rel, flags=flags)
        scratch = torch.empty(max(16, B * S * H * D), dtype=torch.uint8, device=dev)
        ops.encode_tensor("k", k, block, k_rel, km, bits_k, cbk, scale=k_scale, zero=k_zero, stream=k_stream, info=k_info,
                          stream_bytes=k_bytes, flags=flags, scratch=scratch, order=order, order_block=block)
        ops.encode_tensor("v", v, block, v_rel, ops.K_TOKEN, bits_v, cbv, scale=v_scale, zero=v_zero, stream=v_stream, info=v_info,
                          stream_bytes=v_bytes, flags=flags, scratch=scratch, order=order, order_block=block)
        return ops.CompressedLayer(
            k_stream=k_stream, k_info=k_info, k_bytes=k_bytes, k_scale=k_scale, k_zero=k_zero,
            v_stream=v_stream, v_info=v_info, v_bytes=v_bytes, v_scale=v_scale, v_zero=v_zero,
            n_comp=S, kv_heads=H, cbk=cbk, cbv=cbv, bits_k=bits_k, bits_v=bits_v, k_mode=km,
            high_precision_zero=high_precision_zero, order=order)
    if repack_method in (RepackMethod.MEDIAN, RepackMethod.GREEDY):
        kq = ops.quantize(k, block, k_rel, km, bits=bits_k, high_precision_zero=high_precision_zero, flags=flags,
                          scale=k_scale, zero=k_zero)
        vq = ops.quantize(v, block, v_rel, ops.K_TOKEN, bits=bits_v, high_precision_zero=high_precision_zero, flags=flags,
                          scale=v_scale, zero=v_zero)
        order = (ops.median_order(vq.codes, H, block) if repack_method == RepackMethod.MEDIAN
                 else ops.greedy_order(kq.codes, vq.codes, H, block, 16))
        v_scale, v_zero = ops.gather_params(v_scale, order, block, S), ops.gather_params(v_zero, order, block, S)
        if km == ops.K_TOKEN:
            k_scale, k_zero = ops.gather_params(k_scale, order, block, S), ops.gather_params(k_zero, order, block, S)
        ops.encode_codes("k", ops.gather_rows(kq.codes, order, block), cbk, bits_k, stream=k_stream, info=k_info,
                         stream_bytes=k_bytes, flags=flags)
        ops.encode_codes("v", ops.gather_rows(vq.codes, order, block), cbv, bits_v, stream=v_stream, info=v_info,
                         stream_bytes=v_bytes, flags=flags)
        return ops.CompressedLayer(
            k_stream=k_stream, k_info=k_info, k_bytes=k_bytes, k_scale=k_scale, k_zero=k_zero,
            v_stream=v_stream, v_info=v_info, v_bytes=v_bytes, v_scale=v_scale, v_zero=v_zero,
            n_comp=S, kv_heads=H, cbk=cbk, cbv=cbv, bits_k=bits_k, bits_v=bits_v, k_mode=km,
            high_precision_zero=high_precision_zero, order=order)
    scratch = torch.empty(max(16, B * S * H * D), dtype=torch.uint8, device=dev)
    ops.encode_tensor("k", k, block, k_rel, km, bits_k, cbk, scale=k_scale, zero=k_zero, stream=k_stream, info=k_info,
                      stream_bytes=k_bytes, flags=flags, high_precision_zero=high_precision_zero, scratch=scratch)
    ops.encode_tensor("v", v, block, v_rel, ops.K_TOKEN, bits_v, cbv, scale=v_scale, zero=v_zero, stream=v_stream, info=v_info,
                      stream_bytes=v_bytes, flags=flags, high_precision_zero=high_precision_zero, scratch=scratch)
    return ops.CompressedLayer(
        k_stream=k_stream, k_info=k_info, k_bytes=k_bytes, k_scale=k_scale, k_zero=k_zero,
        v_stream=v_stream, v_info=v_info, v_bytes=v_bytes, v_scale=v_scale, v_zero=v_zero,
        n_comp=S, kv_heads=H, cbk=cbk, cbv=cbv, bits_k=bits_k, bits_v=bits_v, k_mode=km,
        high_precision_zero=high_precision_zero)
