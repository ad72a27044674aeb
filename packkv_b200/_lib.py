"""ctypes binding of libpackkv_sm100.so (the C ABI in include/packkv_sm100.h).

There is no fallback: if the shared library is missing the import of any compute entry point
raises, telling the user to build it (``python -m packkv_b200.build``).
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# PACKKV_SM100_LIB: path of another build of the same ABI to load instead of the in-tree one
LIB_PATH = os.environ.get("PACKKV_SM100_LIB") or os.path.join(_PKG, "libpackkv_sm100.so")

PKV_OK, PKV_ERR_BAD_ARGUMENT, PKV_ERR_UNSUPPORTED, PKV_ERR_CUDA, PKV_ERR_TOO_LARGE = 0, 1, 2, 3, 4
STATIC_SCRATCH_BYTES = 16 << 20
FLAG_STREAM_OVERFLOW, FLAG_CODE_RANGE, FLAG_BAD_STREAM, FLAG_TIMEOUT, FLAG_ZERO_RANGE = 1, 2, 4, 8, 16

_i32, _i64, _p, _f32 = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float

_CODEC_ENC = [_p, _i64, _p, _i64, _i64, _p, _i64, _p, _p] + [_i32] * 7 + [_p]
_CODEC_DEC = [_p, _i64, _i64, _p, _i64, _p, _i64, _p] + [_i32] * 7 + [_p]



class AttnArgs(ctypes.Structure):
    """Mirror of pkv_attn_args (include/packkv_sm100.h)."""
    _fields_ = [
        ("q", _p), ("out", _p),
        ("k_stream", _p), ("k_seq_stride", _i64), ("k_capacity", _i64), ("k_info", _p), ("k_info_seq_stride", _i64),
        ("k_scale", _p), ("k_zero", _p),
        ("v_stream", _p), ("v_seq_stride", _i64), ("v_capacity", _i64), ("v_info", _p), ("v_info_seq_stride", _i64),
        ("v_scale", _p), ("v_zero", _p), ("param_blocks", _i32), ("param_tokens", _i32),
        ("k_res", _p), ("v_res", _p), ("res_seq_stride", _i64), ("res_head_stride", _i64),
        ("n_res", _i32), ("batch", _i32), ("kv_heads", _i32), ("group", _i32), ("n_comp", _i32),
        ("cbk", _i32), ("cbv", _i32), ("bits_k", _i32), ("bits_v", _i32),
        ("k_mode", _i32), ("high_precision_zero", _i32), ("is_bf16", _i32), ("scaling", _f32), ("flags", _p),
    ]


class AttnExchange(ctypes.Structure):
    """Mirror of pkv_attn_exchange (include/packkv_sm100.h)."""
    _fields_ = [("n_ranks", _i32), ("rank", _i32), ("gathered", _p * 8), ("arrivals", _p * 8)]


class AttnAppend(ctypes.Structure):
    """Mirror of pkv_attn_append (include/packkv_sm100.h)."""
    _fields_ = [("new_k", _p), ("new_v", _p), ("k_stride_b", _i64), ("k_stride_h", _i64), ("v_stride_b", _i64), ("v_stride_h", _i64),
                ("cos", _p), ("sin", _p), ("cs_stride_b", _i64), ("res_capacity", _i32)]


class AttnPlan(ctypes.Structure):
    """Mirror of pkv_attn_plan (include/packkv_sm100.h)."""
    _fields_ = [("cluster", _i32), ("nsplit", _i32), ("launches", _i32), ("extra", _i32)]


class EncodeArgs(ctypes.Structure):
    """Mirror of pkv_encode_args (include/packkv_sm100.h)."""
    _fields_ = [
        ("x", _p), ("stride_b", _i64), ("stride_h", _i64), ("stride_s", _i64),
        ("scale", _p), ("zero", _p), ("param_blocks", _i32), ("param_tokens", _i32),
        ("stream", _p), ("stream_seq_stride", _i64), ("capacity", _i64),
        ("block_info", _p), ("info_seq_stride", _i64), ("stream_bytes", _p), ("flags", _p),
        ("batch", _i32), ("heads", _i32), ("tokens", _i32), ("first_token", _i32), ("qblock", _i32), ("cb", _i32),
        ("which", _i32), ("bits", _i32), ("mode", _i32), ("high_precision_zero", _i32), ("is_bf16", _i32), ("rel", _f32),
    ]


SIGNATURES = {
    "pkv_encode_tensor": (_i32, [ctypes.POINTER(EncodeArgs), _p, _i64, _p]),
    "pkv_encode_tensor_static": (_i32, [ctypes.POINTER(EncodeArgs), _p]),
    "pkv_encode_tensor_ordered": (_i32, [ctypes.POINTER(EncodeArgs), _p, _i32, _p, _i64, _p]),
    "pkv_value_median_order": (_i32, [ctypes.POINTER(EncodeArgs), _p, _i32, _p]),
    "pkv_kq_mat_vec_mul": (_i32, [_p, _i64, _p, _p, _p] + [_i32] * 6 + [_p, _p]),
    "pkv_wv_mat_vec_mul": (_i32, [_p, _i64, _p, _p, _p] + [_i32] * 6 + [_p, _p]),
    "pkv_fused_kq": (_i32, [_p] * 5 + [_i32] * 4 + [_p]),
    "pkv_fused_wv": (_i32, [_p] * 5 + [_i32] * 4 + [_p]),
    "pkv_median_order": (_i32, [_p, _i64, _p, _p] + [_i32] * 4 + [_p]),
    "pkv_gather_rows": (_i32, [_p, _p, _i64, _p] + [_i32] * 4 + [_p]),
    "pkv_append_residual": (_i32, [_p, _i64, _i64, _i64, _p, _i64, _i64, _i64, _p, _p, _i64, _p, _p, _i64, _i64] + [_i32] * 6 + [_p]),
    "pkv_greedy_order": (_i32, [_p, _p, _i64, _p] + [_i32] * 5 + [_p]),
    "pkv_size_model": (_i32, [_p, _i64] + [_i32] * 4 + [_p, _p, _p]),
    "pkv_gather_params": (_i32, [_p, _p, _i64, _i32, _p] + [_i32] * 3 + [_p]),
    "pkv_rope": (_i32, [_p, _i64, _i64, _i64, _p, _p, _i64, _p, _i64, _i64, _i64] + [_i32] * 5 + [_p]),
    "pkv_dequantize": (_i32, [_p, _i64, _p, _p, _i32, _i32, _i32, _p, _i64, _i64, _i64] + [_i32] * 7 + [_p]),
    "pkv_quantize": (_i32, [_p, _i64, _i64, _i64, _p, _i64, _p, _p] + [_i32] * 8 + [_f32] + [_i32] * 4 + [_p, _p]),
    "pkv_decode_attention": (_i32, [ctypes.POINTER(AttnArgs), _p]),
    "pkv_decode_attention_exchange": (_i32, [ctypes.POINTER(AttnArgs), ctypes.POINTER(AttnExchange), _p]),
    "pkv_decode_attention_append": (_i32, [ctypes.POINTER(AttnArgs), ctypes.POINTER(AttnAppend), ctypes.POINTER(AttnExchange), _p]),
    "pkv_decode_attention_split": (_i32, [ctypes.POINTER(AttnArgs), ctypes.POINTER(AttnAppend), ctypes.POINTER(AttnExchange), ctypes.POINTER(AttnPlan),
                                          _p, _i64, _p]),
    "pkv_attention_plan": (_i32, [ctypes.POINTER(AttnArgs), ctypes.POINTER(AttnPlan), _i64, _i32]),
    "pkv_exchange_wait": (_i32, [_p, _i32, ctypes.c_uint32, ctypes.c_uint32, _p, _p]),
    "pkv_exchange_wait_consume": (_i32, [_p, _i32, ctypes.c_uint32, ctypes.c_uint32, _p, _p]),
    "pkv_exchange_alloc": (_i32, [_i64, ctypes.POINTER(ctypes.c_void_p), _p]),
    "pkv_exchange_free": (_i32, [_p]),
    "pkv_ipc_open": (_i32, [_p, ctypes.POINTER(ctypes.c_void_p)]),
    "pkv_ipc_close": (_i32, [_p]),
    "pkv_abi_version": (_i32, []),
    "pkv_k_encode": (_i32, _CODEC_ENC),
    "pkv_v_encode": (_i32, _CODEC_ENC),
    "pkv_k_decode": (_i32, _CODEC_DEC),
    "pkv_v_decode": (_i32, _CODEC_DEC),
}

_lib = None


class PackKVLibraryError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise PackKVLibraryError(
                f"{LIB_PATH} is missing: build it with `python -m packkv_b200.build` "
                "(nvcc, sm_100a). There is no CPU fallback."
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    """Maps a C-ABI status to the exceptions the reference's callers see."""
    if status == PKV_OK:
        return
    if status == PKV_ERR_UNSUPPORTED:
        raise RuntimeError("not supported")  # same text as the reference's dispatch failure
    if status == PKV_ERR_BAD_ARGUMENT:
        raise ValueError(f"{what}: bad argument")
    if status == PKV_ERR_TOO_LARGE:
        raise ValueError(f"{what}: the call needs more than the {STATIC_SCRATCH_BYTES >> 20} MiB built-in scratch; "
                         "pass your own scratch to encode_tensor instead")
    raise RuntimeError(f"{what}: CUDA error")
