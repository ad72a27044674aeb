"""CPU: the shared library loads without a GPU and exports every entry point that
include/packkv_sm100.h declares; the ctypes table covers the same set.  No compute calls."""
import ctypes
import os
import re

import pytest

from packkv_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    with open(os.path.join(ROOT, "include", "packkv_sm100.h")) as f:
        return sorted(set(re.findall(r"\b(pkv_[a-z0-9_]+)\s*\(", f.read())))


def test_library_exports_every_declared_symbol():
    if not os.path.exists(_lib.LIB_PATH):
        from packkv_b200 import build
        build.build()
    handle = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared()
    assert len(names) >= 14
    for n in names:
        assert hasattr(handle, n), n
    assert sorted(_lib.SIGNATURES) == names
    assert _lib.lib().pkv_abi_version() == 1


def test_argument_blocks_match_the_header_layout():
    # field order of the ctypes mirrors = field order of the C structs
    with open(os.path.join(ROOT, "include", "packkv_sm100.h")) as f:
        text = f.read()
    for cname, ctype in (("pkv_attn_args", _lib.AttnArgs), ("pkv_encode_args", _lib.EncodeArgs)):
        body = re.search(r"typedef struct " + cname + r" \{(.*?)\} " + cname, text, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                fields.append(re.findall(r"[A-Za-z_][A-Za-z0-9_]*", part)[-1])
        assert fields == [n for n, _ in ctype._fields_], cname


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libpackkv_sm100.so")
    with pytest.raises(_lib.PackKVLibraryError):
        _lib.lib()
