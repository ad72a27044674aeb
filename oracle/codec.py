"""ctypes doors onto the CPU codec oracles.  TEST INFRASTRUCTURE ONLY.

``restated`` = oracle/packkv_codec_oracle.c (this repository's plain-C restatement);
``reference`` = oracle/_ref/libpackkv_ref.so (the reference's own sources, compiled by
oracle/build_oracle.py).  Both take and return numpy arrays.  Only tests, the smoke check
and the benchmark's CPU-baseline leg may import this module.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build_oracle

_u8p = ctypes.POINTER(ctypes.c_uint8)
_u32p = ctypes.POINTER(ctypes.c_uint32)


def _ptr(a: np.ndarray, t):
    return a.ctypes.data_as(t)


class _Restated:
    def __init__(self):
        self.lib = ctypes.CDLL(build_oracle.build_restatement())
        for name in ("pkv_oracle_k_encode", "pkv_oracle_v_encode"):
            f = getattr(self.lib, name)
            f.restype = ctypes.c_int64
            f.argtypes = [_u8p, _u8p, _u32p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        for name in ("pkv_oracle_k_decode", "pkv_oracle_v_decode"):
            f = getattr(self.lib, name)
            f.restype = ctypes.c_int
            f.argtypes = [_u8p, _u32p, _u8p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        for name in ("pkv_oracle_k_block_bound", "pkv_oracle_v_block_bound"):
            f = getattr(self.lib, name)
            f.restype = ctypes.c_int64
            f.argtypes = [ctypes.c_int, ctypes.c_int]

    def block_bound(self, which: str, cb: int, bits: int) -> int:
        return int(getattr(self.lib, f"pkv_oracle_{which}_block_bound")(cb, bits))

    def encode(self, which: str, codes: np.ndarray, cb: int, bits: int):
        """codes (ctx, hidden) u8 -> (stream bytes, block_info (n_blocks, 2) u32)."""
        assert codes.dtype == np.uint8 and codes.ndim == 2
        codes = np.ascontiguousarray(codes)
        ctx, hidden = codes.shape
        hb = 128 if which == "k" else 64
        nblk = (ctx // cb) * (hidden // hb)
        out = np.zeros(max(1, nblk * self.block_bound(which, cb, bits)), dtype=np.uint8)
        info = np.zeros((nblk, 2), dtype=np.uint32)
        n = getattr(self.lib, f"pkv_oracle_{which}_encode")(
            _ptr(codes, _u8p), _ptr(out, _u8p), _ptr(info, _u32p), ctx, hidden, cb, hb, bits)
        if n < 0:
            raise ValueError(f"oracle {which}_encode: unsupported arguments ctx={ctx} hidden={hidden} cb={cb} bits={bits}")
        return out[:n].copy(), info

    def decode(self, which: str, stream: np.ndarray, info: np.ndarray, ctx: int, hidden: int, cb: int, bits: int):
        hb = 128 if which == "k" else 64
        stream = np.ascontiguousarray(stream, dtype=np.uint8)
        info = np.ascontiguousarray(info, dtype=np.uint32)
        codes = np.zeros((ctx, hidden), dtype=np.uint8)
        rc = getattr(self.lib, f"pkv_oracle_{which}_decode")(
            _ptr(stream, _u8p), _ptr(info, _u32p), _ptr(codes, _u8p), ctx, hidden, cb, hb, bits)
        if rc != 0:
            raise ValueError(f"oracle {which}_decode: unsupported arguments")
        return codes


class _Reference:
    """The reference's compiled codec.  Instantiated for hidden in {128, 256, 1024}."""

    HIDDEN = (128, 256, 1024)

    def __init__(self, path: str):
        self.lib = ctypes.CDLL(path)
        for name in ("ref_k_encode", "ref_v_encode"):
            f = getattr(self.lib, name)
            f.restype = ctypes.c_longlong
            f.argtypes = [_u8p, _u8p, _u32p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int, ctypes.c_int]
        for name in ("ref_k_decode", "ref_v_decode"):
            f = getattr(self.lib, name)
            f.restype = ctypes.c_longlong
            f.argtypes = [_u8p, _u8p, _u32p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int, ctypes.c_int]

    def supports(self, which: str, hidden: int, cb: int, bits: int) -> bool:
        if hidden not in self.HIDDEN or bits not in (2, 3, 4):
            return False
        return cb in (32, 64, 128) if which == "k" else cb == 128

    def encode(self, which: str, codes: np.ndarray, cb: int, bits: int):
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        ctx, hidden = codes.shape
        hb = 128 if which == "k" else 64
        nblk = (ctx // cb) * (hidden // hb)
        # the reference's callers size the output like the uncompressed codes
        # (evaluation/evaluation.py:426); headers can exceed that for incompressible
        # blocks, so leave head-room.
        out = np.zeros(codes.size * 2 + 4096, dtype=np.uint8)
        info = np.zeros((nblk, 2), dtype=np.uint32)
        n = getattr(self.lib, f"ref_{which}_encode")(
            _ptr(codes, _u8p), _ptr(out, _u8p), _ptr(info, _u32p), ctx, hidden, cb, bits)
        if n < 0:
            raise ValueError("reference codec: combination not instantiated")
        return out[:n].copy(), info

    def decode(self, which: str, stream: np.ndarray, info: np.ndarray, ctx: int, hidden: int, cb: int, bits: int):
        # the reference decoder copies a fixed-size window per block; pad the tail
        stream = np.concatenate([np.ascontiguousarray(stream, dtype=np.uint8), np.zeros(cb * 128, np.uint8)])
        info = np.ascontiguousarray(info, dtype=np.uint32)
        codes = np.zeros((ctx, hidden), dtype=np.uint8)
        rc = getattr(self.lib, f"ref_{which}_decode")(
            _ptr(codes, _u8p), _ptr(stream, _u8p), _ptr(info, _u32p), ctx, hidden, cb, bits)
        if rc != 0:
            raise ValueError("reference codec: combination not instantiated")
        return codes


_restated = None
_reference = None


def restated() -> _Restated:
    global _restated
    if _restated is None:
        _restated = _Restated()
    return _restated


def reference():
    """The compiled reference codec, or None when neither the checkout nor a prebuilt
    oracle/_ref/libpackkv_ref.so is available."""
    global _reference
    if _reference is None:
        path = build_oracle.build_reference()
        if path is None or not os.path.exists(path):
            return None
        _reference = _Reference(path)
    return _reference
