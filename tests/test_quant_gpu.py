"""GPU: the quantiser kernel against the reference's PyTorch arithmetic (restated in
oracle/quant.py, pinned to the reference by tests/test_oracle_quant.py) -- codes, scales and
zero-points bit-exact -- and against the committed golden fixtures."""
import os

import numpy as np
import pytest
import torch

from oracle import quant as Q
from packkv_b200 import ops, synth
from packkv_b200.config import QuantMode

pytestmark = pytest.mark.gpu
MODES = {"channel": QuantMode.ChannelQuant, "token": QuantMode.TokenQuant, "vector": QuantMode.VectorQuant, "block": QuantMode.BlockQuant}


def _bits16(t):
    return t.contiguous().view(torch.int16)


def _check(dev, x, block, rel, mode, hp):
    c, z, s = Q.quant_ints(x, block, rel, mode, hp)
    B, H, S, D = x.shape
    got = ops.quantize(x.to(dev), block, rel, MODES[mode], high_precision_zero=hp)
    torch.cuda.synchronize()
    want_codes = c.flatten(2, 3).permute(0, 2, 1, 3).flatten(2, 3).contiguous().to(torch.uint8)
    assert torch.equal(got.codes.cpu(), want_codes)
    shape = {"channel": (B, H, S // block, D), "token": (B, S), "vector": (B, H, S), "block": (B, S // block)}[mode]
    zs, ss = z.reshape(shape), s.reshape(shape)
    assert torch.equal(_bits16(got.scale.cpu()), _bits16(ss))
    assert torch.equal(_bits16(got.zero.cpu()), _bits16(zs))
    # and back: the dense tensor the reference's cache would hold
    mode_int = {"channel": ops.K_CHANNEL, "token": ops.K_TOKEN, "vector": ops.Q_VECTOR, "block": ops.Q_BLOCK}[mode]
    dense = ops.dequantize(got.codes, got.scale, got.zero, H, block, mode_int, high_precision_zero=hp)
    torch.cuda.synchronize()
    assert torch.equal(_bits16(dense.cpu()), _bits16(Q.dequant(c, z, s, hp)))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("mode", ["channel", "token", "vector", "block"])
def test_bit_exact_against_oracle(cuda_device, dtype, mode):
    k, v = synth.synth_kv(2, 4, 256, 128, seed=21, dtype=dtype, apply_rope=True)
    for x in (k, v):
        for bits in (2, 3, 4):
            for block in (32, 64, 128):
                _check(cuda_device, x, block, synth.rel_for_bits(bits), mode, False)
        for rel in (0.1, 0.2):
            _check(cuda_device, x, 64, rel, mode, False)
        _check(cuda_device, x, 64, 1 / 14, mode, True)


def test_golden_fixtures(cuda_device, golden_dir):
    g = np.load(os.path.join(golden_dir, "quant_golden.npz"))
    for name in g["cases"]:
        dname, mode, bits, blk, hp = str(name).split("_")
        if mode not in MODES:
            continue
        dtype = torch.float16 if dname == "f16" else torch.bfloat16
        x = torch.from_numpy(g[f"{dname}_k"]).view(dtype)
        got = ops.quantize(x.to(cuda_device), int(blk[3:]), synth.rel_for_bits(int(bits[1:])), MODES[mode],
                           high_precision_zero=bool(int(hp[2:])))
        torch.cuda.synchronize()
        c5 = torch.from_numpy(g[f"{name}_codes"])
        want = c5.flatten(2, 3).permute(0, 2, 1, 3).flatten(2, 3).contiguous()
        assert torch.equal(got.codes.cpu(), want), name
        assert np.array_equal(got.scale.cpu().view(torch.int16).numpy().ravel(), g[f"{name}_scale"].ravel()), name
        assert np.array_equal(got.zero.cpu().view(torch.int16).numpy().ravel(), g[f"{name}_zero"].ravel()), name


def test_strided_input_and_range_flag(cuda_device):
    # (B, S, H, D) storage viewed as (B, H, S, D): the layout attention projections produce
    x = torch.randn(2, 128, 4, 128, dtype=torch.float16).transpose(1, 2)
    c, z, s = Q.quant_ints(x, 64, 1 / 14, "token")
    got = ops.quantize(x.to(cuda_device).contiguous().transpose(1, 2).contiguous().transpose(1, 2), 64, 1 / 14, QuantMode.TokenQuant)
    torch.cuda.synchronize()
    assert torch.equal(got.codes.cpu(), c.flatten(2, 3).permute(0, 2, 1, 3).flatten(2, 3).contiguous().to(torch.uint8))
    # rel = 0.1 gives up to 12 levels: does not fit 3 bits -> flagged, not clamped silently
    flags = ops.new_flags(cuda_device)
    ops.quantize(x.to(cuda_device), 64, 0.1, QuantMode.TokenQuant, bits=3, flags=flags)
    torch.cuda.synchronize()
    assert int(flags.item()) & 2
    with pytest.raises(ValueError):
        ops.quantize(x.to(cuda_device)[:, :, :100], 64, 0.1, QuantMode.TokenQuant)


def test_full_size_quantise_pack_round_trip(cuda_device):
    """cfg-sized property: quantise -> pack -> unpack returns the quantiser's codes."""
    k, _ = synth.synth_kv(4, 8, 8192, 128, seed=5, dtype=torch.bfloat16, device=cuda_device, apply_rope=True)
    q = ops.quantize(k, 64, 1 / 14, QuantMode.ChannelQuant, bits=4)
    stream, info, nbytes, flags = ops.encode_codes("k", q.codes, 64, 4)
    back, dflags = ops.decode_codes("k", stream, info, 8192, 1024, 64, 4)
    torch.cuda.synchronize()
    assert int(flags.item()) == 0 and int(dflags.item()) == 0
    assert torch.equal(back, q.codes)
    assert int(q.codes.max().item()) <= 15
