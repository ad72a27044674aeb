"""Device-tensor wrappers over the C ABI (include/packkv_sm100.h).

Everything here takes CUDA tensors, launches on torch's current stream and returns without
synchronising.  Tensors are only the carrier for device memory; the arithmetic is in
libpackkv_sm100.so.
"""
from __future__ import annotations

from typing import Optional, Tuple

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
