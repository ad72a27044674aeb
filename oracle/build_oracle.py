"""Build recipe for the CPU oracle (test infrastructure, never the product).

Two artefacts:

* ``oracle/libpackkv_oracle.so`` -- the plain-C restatement of the bit-pack codec
  (``oracle/packkv_codec_oracle.c``), compiled with gcc.  Always built.
* ``oracle/_ref/libpackkv_ref.so`` -- the reference's own CPU codec
  (``packkv_cuda_ext/src/{k,v}_{encode,decode}_cpu.cpp`` and ``src/utils.cpp``) compiled
  with g++ from where the sources lie in the reference checkout, through
  ``oracle/ref_shim.cpp``.  Built only when the checkout is present (environment variable
  ``PACKKV_REFERENCE`` names it); a prebuilt copy is reused otherwise.
  The reference sources include ``<torch/torch.h>``, so torch's headers and libraries are
  on the compile and link lines; the reference's own build system is not run.

Run ``python oracle/build_oracle.py`` (add ``--force`` to rebuild).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
ORACLE_SO = os.path.join(HERE, "libpackkv_oracle.so")
REF_SO = os.path.join(REF_DIR, "libpackkv_ref.so")


def reference_root() -> str:
    """The reference checkout: $PACKKV_REFERENCE, else a directory `reference` beside this repository."""
    return os.environ.get("PACKKV_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def build_restatement(force: bool = False) -> str:
    src = os.path.join(HERE, "packkv_codec_oracle.c")
    if force or not _newer(ORACLE_SO, src):
        subprocess.check_call(["gcc", "-O2", "-std=c11", "-Wall", "-shared", "-fPIC", src, "-o", ORACLE_SO])
    return ORACLE_SO


def build_reference(force: bool = False) -> str | None:
    """Compile the reference codec; returns the .so path, or None if it cannot be had."""
    ext = os.path.join(reference_root(), "packkv_cuda_ext")
    shim = os.path.join(HERE, "ref_shim.cpp")
    if not os.path.isdir(ext):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, shim):
        return REF_SO
    import torch
    from torch.utils.cpp_extension import include_paths

    os.makedirs(REF_DIR, exist_ok=True)
    incs = [f"-I{ext}", f"-I{os.path.join(ext, 'include')}"] + [f"-I{p}" for p in include_paths()]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    base = ["g++", "-O2", "-std=c++17", "-fPIC", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"] + incs

    def compile_part(part: int) -> str:
        obj = os.path.join(REF_DIR, f"ref_part{part}.o")
        subprocess.check_call(base + [f"-DPART={part}", "-c", shim, "-o", obj])
        return obj

    with ThreadPoolExecutor(max_workers=5) as pool:
        objs = list(pool.map(compile_part, range(1, 6)))
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    subprocess.check_call(
        ["g++", "-shared", "-o", REF_SO] + objs
        + [f"-L{libdir}", f"-Wl,-rpath,{libdir}", "-ltorch", "-ltorch_cpu", "-lc10"]
    )
    return REF_SO


def main() -> None:
    force = "--force" in sys.argv
    print("restatement:", build_restatement(force))
    print("reference  :", build_reference(force))


if __name__ == "__main__":
    main()
