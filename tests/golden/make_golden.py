"""Generates the committed golden fixtures from the REFERENCE itself.

Needs the reference checkout (``PACKKV_REFERENCE``, default: a directory ``reference`` beside this repository): its
``utils/compute.py`` is imported for the quantiser / reorder / size model, and its CPU
codec sources are compiled by ``oracle/build_oracle.py``.  Run from the repository root:

    python tests/golden/make_golden.py

Outputs (small, committed):
  codec_golden.npz   seeded code matrices and the reference's streams / block_info
  quant_golden.npz   seeded fp16/bf16 K,V (raw bit patterns) and the reference's codes,
                     zero-points, scales, median order and size-model bytes
  cfg0_digest.json   SHA-256 digests of every stage of the seq-1024 configuration (inputs
                     are regenerated from the seed at test time; their digest is included)
"""
from __future__ import annotations

import hashlib
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
REF = os.environ.get("PACKKV_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
sys.path.insert(0, REF)

from oracle import codec  # noqa: E402
from packkv_b200 import synth  # noqa: E402
from utils import compute as ref  # noqa: E402  (the reference's module)

HERE = os.path.dirname(os.path.abspath(__file__))
MODES = {"channel": ref.QuantMode.ChannelQuant, "token": ref.QuantMode.TokenQuant,
         "vector": ref.QuantMode.VectorQuant, "block": ref.QuantMode.BlockQuant}


def sha(a) -> str:
    if isinstance(a, torch.Tensor):
        a = a.contiguous().view(torch.uint8).numpy() if a.dtype != torch.uint8 else a.contiguous().numpy()
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def code_matrix(rng, kind: int, ctx: int, hidden: int, bits: int) -> np.ndarray:
    top = 2 ** bits
    if kind == 0:
        return rng.integers(0, top, (ctx, hidden), dtype=np.uint8)
    if kind == 1:
        return np.clip(np.round(rng.normal(top / 2, 1.0, (ctx, hidden))), 0, top - 1).astype(np.uint8)
    if kind == 2:
        return np.clip(np.round(rng.normal(top / 2, 0.4, (ctx, hidden))), 0, top - 1).astype(np.uint8)
    return np.full((ctx, hidden), top - 1, dtype=np.uint8)


def make_codec():
    refc = codec.reference()
    assert refc is not None, "reference codec not built"
    rng = np.random.default_rng(20240)
    out = {}
    cases = []
    for which, cb, bits, hidden in [("k", 64, 4, 256), ("k", 64, 3, 128), ("k", 128, 2, 128), ("k", 32, 4, 128),
                                    ("k", 32, 3, 256), ("v", 128, 3, 128), ("v", 128, 4, 256), ("v", 128, 2, 128)]:
        for kind in range(4):
            ctx = 2 * cb if cb < 128 else cb
            codes = code_matrix(rng, kind, ctx, hidden, bits)
            stream, info = refc.encode(which, codes, cb, bits)
            assert (refc.decode(which, stream, info, ctx, hidden, cb, bits) == codes).all()
            name = f"{which}_cb{cb}_b{bits}_h{hidden}_d{kind}"
            out[name + "_codes"], out[name + "_stream"], out[name + "_info"] = codes, stream, info
            cases.append(name)
    out["cases"] = np.array(cases)
    np.savez_compressed(os.path.join(HERE, "codec_golden.npz"), **out)


def make_quant():
    out = {}
    cases = []
    for dtype, dname in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        k, v = synth.synth_kv(1, 2, 128, 128, seed=11, dtype=dtype, apply_rope=True)
        out[f"{dname}_k"], out[f"{dname}_v"] = bits16(k), bits16(v)
        for mode, m in MODES.items():
            for bits in (2, 3, 4):
                for block in (32, 64):
                    rel = synth.rel_for_bits(bits)
                    for hp in (False, True):
                        c, z, s = ref.quant_ints(k, block, rel, m, hp)
                        name = f"{dname}_{mode}_b{bits}_blk{block}_hp{int(hp)}"
                        out[name + "_codes"] = c.to(torch.uint8).numpy()
                        out[name + "_zero"], out[name + "_scale"] = bits16(z), bits16(s)
                        cases.append(name)
        # reorder + size model on the north-star pairing (K channel, V token), 4 bit, block 64
        kc, _, _ = ref.quant_ints(k, 64, 1 / 14, MODES["channel"])
        vc, _, _ = ref.quant_ints(v, 64, 1 / 14, MODES["token"])
        blocks = torch.cat([kc.permute(2, 3, 0, 1, 4).flatten(2, 4), vc.permute(2, 3, 0, 1, 4).flatten(2, 4)], dim=2)
        re = ref.median_repacking(blocks)
        out[f"{dname}_median_blocks"] = re.to(torch.uint8).numpy()
        out[f"{dname}_sizes"] = np.array(ref.repack_and_encode(kc, vc, 16, ref.RepackMethod.MEDIAN), dtype=np.int64)
        out[f"{dname}_greedy_blocks"] = ref.greedy_repacking(blocks, 16).to(torch.uint8).numpy()
        out[f"{dname}_greedy_sizes"] = np.array(ref.repack_and_encode(kc, vc, 16, ref.RepackMethod.GREEDY), dtype=np.int64)
    out["cases"] = np.array(cases)
    np.savez_compressed(os.path.join(HERE, "quant_golden.npz"), **out)


def make_cfg0():
    """seq-1024 plumbing configuration: (1,8,1024,128) fp16, seed 0, block 64."""
    refc = codec.reference()
    k, v = synth.synth_kv(1, 8, 1024, 128, seed=0, dtype=torch.float16, apply_rope=False)
    d = {"k_input": sha(k), "v_input": sha(v)}
    for tag, x, mode, rel, which, cb, bits in [
        ("k_channel_b4", k, "channel", 1 / 14, "k", 64, 4),
        ("k_token_b4", k, "token", 1 / 14, "k", 64, 4),
        ("k_token_rel0.1", k, "token", 0.1, "k", 64, 4),
        ("v_token_b4", v, "token", 1 / 14, "v", 128, 4),
        ("v_token_rel0.2", v, "token", 0.2, "v", 128, 3),
    ]:
        c, z, s = ref.quant_ints(x, 64, rel, MODES[mode])
        mat = c.flatten(2, 3).permute(2, 0, 1, 3).flatten(1, 3).contiguous().to(torch.uint8).numpy()
        stream, info = refc.encode(which, mat, cb, bits)
        d[tag] = {"codes": sha(mat), "zero": sha(z), "scale": sha(s), "stream": sha(stream), "info": sha(info),
                  "stream_bytes": int(stream.size), "max_code": int(mat.max())}
    with open(os.path.join(HERE, "cfg0_digest.json"), "w") as f:
        json.dump(d, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    make_codec()
    make_quant()
    make_cfg0()
    for n in ("codec_golden.npz", "quant_golden.npz", "cfg0_digest.json"):
        print(n, os.path.getsize(os.path.join(HERE, n)), "bytes")
