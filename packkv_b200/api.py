"""The reference's ``packkv_cuda`` entry points (packkv_cuda_ext/packkv_cuda.pyi:4-86,
export_packkv.cpp:9-18), same names and positional arguments, on the B200 kernels.

Differences a caller can observe, all deliberate:
* the four ``*_cpu`` codec functions still accept CPU tensors (they are staged through device
  memory; there is no CPU arithmetic in this package) and also accept CUDA tensors directly;
* more shapes are accepted than the reference dispatches (bits 2..4, K token blocks 32/64/128,
  V token blocks 32/64/128, any hidden_dim that is a multiple of the block width); anything else
  raises ``RuntimeError("not supported")`` exactly like the reference;
* contract violations raise ``ValueError`` instead of aborting the process;
* the four GPU functions run on torch's current stream; they still return elapsed milliseconds
  (CUDA events around the launch, then a synchronise), which makes them benchmark helpers just
  like the reference's.
"""
from __future__ import annotations

import torch

from . import _lib, ops

_U32 = getattr(torch, "uint32", torch.int32)


def _dev() -> torch.device:
    if not torch.cuda.is_available():
        raise _lib.PackKVLibraryError("packkv_cuda needs a CUDA device: there is no CPU fallback")
    return torch.device("cuda", torch.cuda.current_device())


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(f"PackKV Assertion failed: {msg}")


def _check_codec_args(which, codes, compressed, info, ctx_len, hidden_dim, cb, hb, bits):
    # the reference's asserts (k_encode_cpu.cpp:248-284, v_encode_cpu.cpp:263-299)
    _require(codes.dim() == 2 and codes.size(0) == ctx_len, "ctx_len mismatch")
    _require(codes.size(1) == hidden_dim, "hidden_dim mismatch")
    _require(cb > 0 and hb > 0, "block sizes must be greater than 0")
    _require(ctx_len % cb == 0, "ctx_len must be divisible by ctx_len_block_size")
    _require(hidden_dim % hb == 0, "hidden_dim must be divisible by hidden_dim_block_size")
    nblk = (ctx_len // cb) * (hidden_dim // hb)
    _require(info.dim() == 2 and info.size(0) == nblk, "block_info_buffer block num mismatch")
    _require(info.size(1) == 2, "block_info_buffer.size(1) must be 2")
    _require(bits <= 4, "bits_len must be less than or equal to 4")
    _require(cb % 16 == 0, "ctx_len_block_size must be divisible by PACK_ELE_NUM")
    if which == "k":
        _require(hb == 128, "hidden_dim_block_size must be 128, because this is most common head dim")
    _require(codes.dtype == torch.uint8, "quant_ints_tensor must be a UInt8 tensor")
    _require(compressed.dtype == torch.uint8, "compressed_buffer must be a UInt8 tensor")
    _require(compressed.numel() > 0, "compressed_buffer must be a non-empty tensor")
    _require(info.dtype in (_U32, torch.int32), "block_info_buffer must be a UInt32 tensor")
    _require(codes.is_contiguous() and compressed.is_contiguous() and info.is_contiguous(), "tensors must be contiguous")
    if which == "v" and hb != 64:
        raise RuntimeError("not supported")


def _encode(which, codes, compressed, info, ctx_len, hidden_dim, cb, hb, bits) -> int:
    _check_codec_args(which, codes, compressed, info, ctx_len, hidden_dim, cb, hb, bits)
    dev = codes.device if codes.is_cuda else _dev()
    d_codes = codes.to(dev).unsqueeze(0)
    staged = not compressed.is_cuda
    cap = compressed.numel()
    d_stream = (torch.zeros(cap + 16, dtype=torch.uint8, device=dev) if staged else compressed.view(-1)).unsqueeze(0)
    d_info = (torch.zeros(info.shape, dtype=torch.int32, device=dev) if not info.is_cuda else info.view(torch.int32)).unsqueeze(0)
    flags = ops.new_flags(dev)
    nbytes = torch.zeros(1, dtype=torch.int32, device=dev)
    fn = _lib.lib().pkv_k_encode if which == "k" else _lib.lib().pkv_v_encode
    st = fn(d_codes.data_ptr(), d_codes.stride(0), d_stream.data_ptr(), d_stream.stride(0), cap,
            d_info.data_ptr(), d_info.shape[1], nbytes.data_ptr(), flags.data_ptr(),
            1, ctx_len, hidden_dim, cb, hb, bits, 0, ops._stream_ptr())
    _lib.check(st, f"{which}_encode_cpu")
    f = int(flags.item())   # synchronises
    if f & _lib.FLAG_STREAM_OVERFLOW:
        raise ValueError("compressed_buffer is too small for the encoded stream")
    if f & _lib.FLAG_CODE_RANGE:
        raise ValueError(f"quant_ints_tensor holds codes that do not fit {bits} bits")
    total = int(nbytes.item())
    if staged:
        compressed.view(-1)[:total].copy_(d_stream[0, :total])
    if not info.is_cuda:
        info.view(torch.int32).copy_(d_info[0])
    return total


def _decode(which, compressed, info, codes, ctx_len, hidden_dim, cb, hb, bits) -> None:
    _check_codec_args(which, codes, compressed, info, ctx_len, hidden_dim, cb, hb, bits)
    dev = compressed.device if compressed.is_cuda else _dev()
    flat = compressed.reshape(-1)
    d_stream = torch.zeros((flat.numel() + 31) // 16 * 16, dtype=torch.uint8, device=dev)
    d_stream[: flat.numel()].copy_(flat)
    d_info = info.view(torch.int32).to(dev).unsqueeze(0)
    d_codes = codes if codes.is_cuda else torch.zeros(codes.shape, dtype=torch.uint8, device=dev)
    flags = ops.new_flags(dev)
    fn = _lib.lib().pkv_k_decode if which == "k" else _lib.lib().pkv_v_decode
    st = fn(d_stream.data_ptr(), d_stream.numel(), flat.numel(), d_info.data_ptr(), d_info.shape[1],
            d_codes.data_ptr(), d_codes.numel(), flags.data_ptr(), 1, ctx_len, hidden_dim, cb, hb, bits, 0, ops._stream_ptr())
    _lib.check(st, f"{which}_decode_cpu")
    if int(flags.item()) & _lib.FLAG_BAD_STREAM:
        raise ValueError("block_info_buffer / compressed_buffer are inconsistent")
    if not codes.is_cuda:
        codes.copy_(d_codes)


def k_encode_cpu(quant_ints_tensor, compressed_buffer, block_info_buffer, ctx_len, hidden_dim,
                 ctx_len_block_size, hidden_dim_block_size, bits_len) -> int:
    return _encode("k", quant_ints_tensor, compressed_buffer, block_info_buffer, ctx_len, hidden_dim,
                   ctx_len_block_size, hidden_dim_block_size, bits_len)


def v_encode_cpu(quant_ints_tensor, compressed_buffer, block_info_buffer, ctx_len, hidden_dim,
                 ctx_len_block_size, hidden_dim_block_size, bits_len) -> int:
    return _encode("v", quant_ints_tensor, compressed_buffer, block_info_buffer, ctx_len, hidden_dim,
                   ctx_len_block_size, hidden_dim_block_size, bits_len)


def k_decode_cpu(compressed_buffer, block_info_buffer, quant_ints_tensor, ctx_len, hidden_dim,
                 ctx_len_block_size, hidden_dim_block_size, bits_len) -> None:
    _decode("k", compressed_buffer, block_info_buffer, quant_ints_tensor, ctx_len, hidden_dim,
            ctx_len_block_size, hidden_dim_block_size, bits_len)


def v_decode_cpu(compressed_buffer, block_info_buffer, quant_ints_tensor, ctx_len, hidden_dim,
                 ctx_len_block_size, hidden_dim_block_size, bits_len) -> None:
    _decode("v", compressed_buffer, block_info_buffer, quant_ints_tensor, ctx_len, hidden_dim,
            ctx_len_block_size, hidden_dim_block_size, bits_len)


def _timed(launch) -> float:
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    launch()
    end.record()
    end.synchronize()
    return start.elapsed_time(end)


def _matvec(which, compressed, info, vec, out, ctx_len, hidden_dim, cb, hb, bits) -> float:
    for t in (compressed, info, vec, out):
        _require(t.is_cuda, "tensors must be CUDA tensors")
    if vec.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("not supported")   # the reference prints "Unsupported data type" and returns 0.0
    _require(vec.is_contiguous() and out.is_contiguous() and info.is_contiguous(), "tensors must be contiguous")
    heads = hidden_dim // 128
    if which == "k":
        _require(vec.numel() == heads * 128 and out.numel() == heads * ctx_len and out.dtype == vec.dtype, "q / kq_out shape")
    else:
        _require(vec.numel() == heads * ctx_len and out.numel() == hidden_dim and out.dtype == torch.float32, "w / wv_out shape")
    flat = compressed.reshape(-1)
    if flat.data_ptr() % 16:
        flat = flat.clone()
    flags = ops.new_flags(vec.device)
    fn = _lib.lib().pkv_kq_mat_vec_mul if which == "k" else _lib.lib().pkv_wv_mat_vec_mul
    status = []
    ms = _timed(lambda: status.append(fn(flat.data_ptr(), flat.numel(), info.data_ptr(), vec.data_ptr(), out.data_ptr(),
                                         ctx_len, hidden_dim, cb, hb, bits, int(vec.dtype == torch.bfloat16),
                                         flags.data_ptr(), ops._stream_ptr())))
    _lib.check(status[0], f"{which}_mat_vec_mul")
    if int(flags.item()):
        raise ValueError("block_info_buffer / compressed_buffer are inconsistent")
    return ms


def kq_mat_vec_mul(compressed_buffer, block_info_buffer, q, kq_out, ctx_len, hidden_dim,
                   ctx_len_block_size, hidden_dim_block_size, bits_len) -> float:
    return _matvec("k", compressed_buffer, block_info_buffer, q, kq_out, ctx_len, hidden_dim,
                   ctx_len_block_size, hidden_dim_block_size, bits_len)


def wv_mat_vec_mul(compressed_buffer, block_info_buffer, w, wv_out, ctx_len, hidden_dim,
                   ctx_len_block_size, hidden_dim_block_size, bits_len) -> float:
    return _matvec("v", compressed_buffer, block_info_buffer, w, wv_out, ctx_len, hidden_dim,
                   ctx_len_block_size, hidden_dim_block_size, bits_len)


def _epilogue(is_kq, out, a, zero, scale, t) -> float:
    for x in (out, a, zero, scale, t):
        if not x.is_cuda or not x.is_contiguous():
            raise ValueError("tensors must be contiguous CUDA tensors")
    if a.dtype not in (torch.float16, torch.bfloat16) or any(x.dtype != a.dtype for x in (out, zero, scale, t)):
        raise ValueError("all tensors must share one dtype, fp16 or bf16")
    M, inner = a.shape
    N = zero.numel()
    if is_kq:
        if tuple(t.shape) != (M, N) or tuple(out.shape) != (M, N) or scale.numel() != N:
            raise ValueError("fused_kq: shape mismatch")
        args = (M, N, inner)
        fn = _lib.lib().pkv_fused_kq
    else:
        if inner != N or scale.numel() != N or t.shape[0] != M or tuple(out.shape) != tuple(t.shape):
            raise ValueError("fused_wv: shape mismatch")
        args = (M, N, t.shape[1])
        fn = _lib.lib().pkv_fused_wv
    status = []
    ms = _timed(lambda: status.append(fn(out.data_ptr(), a.data_ptr(), zero.data_ptr(), scale.data_ptr(), t.data_ptr(),
                                         *args, int(a.dtype == torch.bfloat16), ops._stream_ptr())))
    _lib.check(status[0], "fused_kq" if is_kq else "fused_wv")
    return ms


def fused_kq(our_kq, q, k_quant_zero, k_quant_scale, t) -> float:
    return _epilogue(True, our_kq, q, k_quant_zero, k_quant_scale, t)


def fused_wv(our_wv, w, v_quant_zero, v_quant_scale, term1) -> float:
    return _epilogue(False, our_wv, w, v_quant_zero, v_quant_scale, term1)
