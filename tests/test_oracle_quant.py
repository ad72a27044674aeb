"""CPU: the quantiser / reorder / size-model / attention restatement (oracle/quant.py) against
the committed golden vectors made from the reference's utils/compute.py, and against that
module itself when the reference checkout is present."""
import hashlib
import json
import os
import sys

import numpy as np
import pytest
import torch

from oracle import codec
from oracle import quant as Q
from packkv_b200 import synth

REF = os.environ.get("PACKKV_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


def _sha(a):
    if isinstance(a, torch.Tensor):
        a = a.contiguous().view(torch.uint8).numpy() if a.dtype != torch.uint8 else a.contiguous().numpy()
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.fixture(scope="module")
def golden(golden_dir):
    return np.load(os.path.join(golden_dir, "quant_golden.npz"))


def test_quantiser_matches_golden(golden):
    for name in golden["cases"]:
        dname, mode, bits, blk, hp = str(name).split("_")
        dtype = torch.float16 if dname == "f16" else torch.bfloat16
        x = torch.from_numpy(golden[f"{dname}_k"]).view(dtype)
        c, z, s = Q.quant_ints(x, int(blk[3:]), synth.rel_for_bits(int(bits[1:])), mode, bool(int(hp[2:])))
        assert np.array_equal(c.to(torch.uint8).numpy(), golden[f"{name}_codes"]), name
        assert np.array_equal(z.contiguous().view(torch.int16).numpy(), golden[f"{name}_zero"]), name
        assert np.array_equal(s.contiguous().view(torch.int16).numpy(), golden[f"{name}_scale"]), name


def test_median_reorder_and_size_model_match_golden(golden):
    for dname, dtype in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        k = torch.from_numpy(golden[f"{dname}_k"]).view(dtype)
        v = torch.from_numpy(golden[f"{dname}_v"]).view(dtype)
        kc, _, _ = Q.quant_ints(k, 64, 1 / 14, "channel")
        vc, _, _ = Q.quant_ints(v, 64, 1 / 14, "token")
        blocks = Q.kv_feature_blocks(kc, vc)
        re = Q.median_reorder(blocks)
        assert np.array_equal(re.to(torch.uint8).numpy(), golden[f"{dname}_median_blocks"])
        pre, aft = Q.size_model(blocks, 16), Q.size_model(re, 16)
        assert list(golden[f"{dname}_sizes"]) == [pre[0], pre[1], aft[0], aft[1]]


def test_greedy_reorder_matches_golden(golden):
    for dname, dtype in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        k = torch.from_numpy(golden[f"{dname}_k"]).view(dtype)
        v = torch.from_numpy(golden[f"{dname}_v"]).view(dtype)
        kc, _, _ = Q.quant_ints(k, 64, 1 / 14, "channel")
        vc, _, _ = Q.quant_ints(v, 64, 1 / 14, "token")
        blocks = Q.kv_feature_blocks(kc, vc)
        re = Q.greedy_reorder(blocks, 16)
        assert np.array_equal(re.to(torch.uint8).numpy(), golden[f"{dname}_greedy_blocks"])
        pre, aft = Q.size_model(blocks, 16), Q.size_model(re, 16)
        assert list(golden[f"{dname}_greedy_sizes"]) == [pre[0], pre[1], aft[0], aft[1]]


def test_cfg0_digests(golden_dir):
    """seq-1024 plumbing configuration, every stage, by SHA-256."""
    with open(os.path.join(golden_dir, "cfg0_digest.json")) as f:
        want = json.load(f)
    k, v = synth.synth_kv(1, 8, 1024, 128, seed=0, dtype=torch.float16, apply_rope=False)
    assert _sha(k) == want["k_input"] and _sha(v) == want["v_input"], "seeded generator drifted"
    R = codec.restated()
    for tag, x, mode, rel, which, cb, bits in [
        ("k_channel_b4", k, "channel", 1 / 14, "k", 64, 4), ("k_token_b4", k, "token", 1 / 14, "k", 64, 4),
        ("k_token_rel0.1", k, "token", 0.1, "k", 64, 4), ("v_token_b4", v, "token", 1 / 14, "v", 128, 4),
        ("v_token_rel0.2", v, "token", 0.2, "v", 128, 3),
    ]:
        c, z, s = Q.quant_ints(x, 64, rel, mode)
        mat = Q.codes_matrix(c).numpy()
        stream, info = R.encode(which, mat, cb, bits)
        w = want[tag]
        assert (_sha(mat), _sha(z), _sha(s), _sha(stream), _sha(info)) == (w["codes"], w["zero"], w["scale"], w["stream"], w["info"]), tag
        assert stream.size == w["stream_bytes"] and int(mat.max()) == w["max_code"]
        assert np.array_equal(R.decode(which, stream, info, 1024, 1024, cb, bits), mat)


def test_cache_state_machine_lengths():
    for L in range(1, 600):
        n = Q.compress_block_count(L, 64, 192)
        assert n == max(0, (L + 64 - L % 64 - 192) // 64)
        assert L - 64 * n <= 191
    layer = Q.CacheLayerOracle(64, 192, 1 / 14, 1 / 14, "channel", "token")
    cos, sin = synth.rope_tables(300, 128, dtype=torch.float16)
    k, v = synth.synth_kv(1, 2, 300, 128, seed=3, dtype=torch.float16)
    K, V = layer.update(k, v, cos, sin)
    assert K.shape[2] == 300 and layer.k_res.shape[2] == 300 - 128 and layer.seq_length() == 300
    for step in range(70):
        cos1, sin1 = synth.rope_tables(1, 128, start=300 + step, dtype=torch.float16)
        K, V = layer.update(k[:, :, :1], v[:, :, :1], cos1, sin1)
        assert 128 <= layer.k_res.shape[2] <= 191
    assert layer.seq_length() == 370


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "utils")), reason="reference checkout not present")
def test_against_imported_reference():
    sys.path.insert(0, REF)
    try:
        from utils import compute as ref
    finally:
        sys.path.remove(REF)
    modes = {"block": ref.QuantMode.BlockQuant, "channel": ref.QuantMode.ChannelQuant,
             "token": ref.QuantMode.TokenQuant, "vector": ref.QuantMode.VectorQuant}
    for dtype in (torch.float16, torch.bfloat16):
        k, v = synth.synth_kv(2, 2, 256, 128, seed=8, dtype=dtype, apply_rope=True)
        for name, m in modes.items():
            for rel in (0.1, 1 / 14, 1 / 2):
                for hp in (False, True):
                    for a, b in zip(ref.quant_ints(k, 64, rel, m, hp), Q.quant_ints(k, 64, rel, name, hp)):
                        assert torch.equal(a, b)
        kc, _, _ = Q.quant_ints(k, 64, 1 / 14, "channel")
        vc, _, _ = Q.quant_ints(v, 64, 1 / 14, "token")
        blocks = Q.kv_feature_blocks(kc, vc)
        assert torch.equal(ref.median_repacking(blocks), Q.median_reorder(blocks))
        assert ref.repack_and_encode(kc, vc, 16, ref.RepackMethod.MEDIAN)[2:] == Q.size_model(Q.median_reorder(blocks), 16)
        assert torch.equal(ref.greedy_repacking(blocks, 16).to(blocks.dtype), Q.greedy_reorder(blocks, 16))
        cos, sin = synth.rope_tables(256, 128, dtype=dtype)
        assert torch.equal(ref.apply_rotary_pos_emb_single(k, cos, sin), Q.rope(k, cos, sin))
        # cache step: cut + quantise + dequantise + cat
        hist, res = ref.quant_error(None, None, k, 64, 192, 1 / 14, ref.QuantMode.ChannelQuant)
        layer = Q.CacheLayerOracle(64, 192, 1 / 14, 1 / 14, "channel", "token")
        h2, r2 = layer._step(None, None, k, 1 / 14, "channel")
        assert torch.equal(hist, h2) and torch.equal(res, r2)
