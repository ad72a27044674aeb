"""GPU: fused decompress-attention decode (C ABI pkv_decode_attention) against the
reference's decompress-then-attend path restated on CPU (oracle/quant.py): quantise ->
dequantise in the tensor dtype -> eager attention with fp32 softmax.

Tolerance: 2e-3 max-abs error relative to max|reference| (the bar of the task), both dtypes.
"""
import pytest
import torch

from oracle import quant as Q
from packkv_b200 import ops, synth
from tests.helpers import layer_from_oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _run_case(dev, dtype, B, Hkv, G, n_comp, n_res, *, block, cbk, cbv, bits_k, bits_v, k_mode, seed, hp=False, rope=True, plan=None, scratch=None,
              repeats=1):
    S = n_comp + n_res
    k, v = synth.synth_kv(B, Hkv, S, 128, seed=seed, dtype=dtype, apply_rope=rope)
    q = synth.synth_q(B, Hkv * G, 128, seed=seed, dtype=dtype)
    layer = kd = vd = None
    if n_comp:
        layer, kd, vd = layer_from_oracle(k[:, :, :n_comp], v[:, :, :n_comp], block=block, bits_k=bits_k, bits_v=bits_v,
                                          k_mode=k_mode, cbk=cbk, cbv=cbv, rel_k=synth.rel_for_bits(bits_k),
                                          rel_v=synth.rel_for_bits(bits_v), device=dev, hp=hp)
    K = k[:, :, n_comp:] if kd is None else torch.cat([kd, k[:, :, n_comp:]], 2)
    V = v[:, :, n_comp:] if vd is None else torch.cat([vd, v[:, :, n_comp:]], 2)
    ref = Q.eager_attention(q, K, V)[:, 0].float()           # (B, Hq, D)
    k_res = k[:, :, n_comp:].contiguous().to(dev) if n_res else None
    v_res = v[:, :, n_comp:].contiguous().to(dev) if n_res else None
    flags = ops.new_flags(dev)
    if plan is not None and scratch is None:
        scratch = ops.new_attention_scratch(dev)
    qd = q[:, :, 0].contiguous().to(dev)
    for _ in range(repeats):                                 # the scratch's counters must come back to zero every time
        out = ops.decode_attention(qd, layer, k_res, v_res, n_res, flags=flags, kv_heads=Hkv, plan=plan, scratch=scratch)
    torch.cuda.synchronize()
    assert int(flags.item()) == 0
    return _rel_err(out.float().cpu(), ref, dtype)


def _rel_err(out, ref, dtype):
    """max |out - ref| / max |ref|.  The output is rounded to the element type once, at the very end, from an fp32
    sum whose order differs from the reference's; when the exact value sits on a rounding boundary the two
    roundings can land on neighbouring values, and one unit in the last place of an element near the maximum
    is already 2^-8 .. 2^-7 of the maximum, above the bar.  Up to two such elements (off by exactly one unit in
    the last place of their own magnitude) are left out of the maximum; anything else counts."""
    diff, top = (out - ref).abs(), ref.abs().max()
    err = (diff.max() / top).item()
    if err > TOL:
        mant = 7 if dtype == torch.bfloat16 else 10
        ulp = torch.exp2(torch.floor(torch.log2(ref.abs().clamp_min(1e-30))) - mant)
        over = diff > TOL * top
        if int(over.sum()) <= 2 and bool((diff[over] <= ulp[over] * 1.0001).all()):
            err = (diff[~over].max() / top).item()
    return err


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("k_mode", ["channel", "token"])
def test_gqa_4bit_block64(cuda_device, dtype, k_mode):
    err = _run_case(cuda_device, dtype, 2, 2, 4, 512, 128, block=64, cbk=64, cbv=64, bits_k=4, bits_v=4, k_mode=k_mode, seed=1)
    assert err <= TOL, err


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_v_block_128_reference_layout(cuda_device, dtype):
    err = _run_case(cuda_device, dtype, 1, 8, 4, 1024 - 128, 128, block=64, cbk=64, cbv=128, bits_k=4, bits_v=4, k_mode="channel", seed=0, rope=False)
    assert err <= TOL, err


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_long_context_2bit_k_block128(cuda_device, dtype):
    err = _run_case(cuda_device, dtype, 1, 2, 4, 2048, 160, block=128, cbk=128, cbv=128, bits_k=2, bits_v=4, k_mode="channel", seed=2)
    assert err <= TOL, err


@pytest.mark.parametrize("G", [1, 2, 8])
def test_group_sizes(cuda_device, G):
    err = _run_case(cuda_device, torch.float16, 2, 2, G, 256, 130, block=64, cbk=64, cbv=64, bits_k=3, bits_v=3, k_mode="token", seed=3)
    assert err <= TOL, err


def test_residual_only_and_compressed_only(cuda_device):
    err = _run_case(cuda_device, torch.float16, 2, 2, 4, 0, 191, block=64, cbk=64, cbv=64, bits_k=4, bits_v=4, k_mode="channel", seed=4)
    assert err <= TOL, err
    err = _run_case(cuda_device, torch.bfloat16, 1, 2, 4, 384, 0, block=64, cbk=64, cbv=64, bits_k=4, bits_v=4, k_mode="channel", seed=5)
    assert err <= TOL, err


def test_high_precision_zero_point(cuda_device):
    err = _run_case(cuda_device, torch.float16, 1, 2, 4, 256, 128, block=64, cbk=64, cbv=64, bits_k=4, bits_v=4, k_mode="channel", seed=6, hp=True)
    assert err <= TOL, err


def test_permutation_invariance(cuda_device):
    """Attention over the compressed tokens does not depend on the token order inside a
    block, the property the reorder step relies on (models/cache/unorder_cache.py:11-20)."""
    dev, dtype = cuda_device, torch.float16
    B, H, G, S = 1, 2, 4, 256
    k, v = synth.synth_kv(B, H, S, 128, seed=9, dtype=dtype)
    q = synth.synth_q(B, H * G, 128, seed=9, dtype=dtype)[:, :, 0].contiguous().to(dev)
    outs = []
    g = torch.Generator().manual_seed(0)
    for shuffle in (False, True):
        kk, vv = k, v
        if shuffle:   # K token-mode and V token-mode parameters travel with their token
            perm = torch.cat([torch.randperm(64, generator=g) + 64 * i for i in range(S // 64)])
            kk, vv = k[:, :, perm], v[:, :, perm]
        layer, _, _ = layer_from_oracle(kk, vv, block=64, bits_k=4, bits_v=4, k_mode="token", cbk=64, cbv=64,
                                        rel_k=1 / 14, rel_v=1 / 14, device=dev)
        outs.append(ops.decode_attention(q, layer, None, None, 0).float().cpu())
    torch.cuda.synchronize()
    assert ((outs[0] - outs[1]).abs().max() / outs[0].abs().max()).item() <= TOL


@pytest.mark.parametrize("shape", [
    # (B, Hkv, G, n_comp, n_res, block, bits_k, bits_v, dtype): the decode configurations of the benchmark at full size
    (16, 8, 4, 8064, 128, 64, 4, 4, torch.bfloat16),
    (8, 8, 4, 32640, 128, 128, 2, 4, torch.bfloat16),
])
def test_full_size_weights_sum_to_one(cuda_device, shape):
    """Size-independent property at the benchmark's sizes: if every token carries the same V row,
    the output is that row whatever the scores are (the probabilities sum to one).  Compressed
    tokens contribute the dequantised row d, residual tokens the original row v, so every output
    element lies between d and v (up to the rounding tolerance); with no residual it equals d.
    Every probability is rounded to the element type (as in the reference), so their sum is one
    only up to a relative 2^-8: that slack is part of the bound."""
    from packkv_b200 import encode
    from packkv_b200.config import QuantMode
    B, Hkv, G, n_comp, n_res, block, bits_k, bits_v, dtype = shape
    dev = cuda_device
    g = torch.Generator().manual_seed(41)
    k, _ = synth.synth_kv(B, Hkv, n_comp + n_res, 128, seed=41, dtype=dtype, device=dev, apply_rope=True)
    v_row = torch.randn(B, Hkv, 1, 128, generator=g).to(dtype)
    q = synth.synth_q(B, Hkv * G, 128, seed=41, dtype=dtype)[:, :, 0].contiguous().to(dev)
    rel_v = synth.rel_for_bits(bits_v)
    # the dequantised row, from the oracle on one block of identical tokens
    vc, vz, vs = Q.quant_ints(v_row.expand(B, Hkv, block, 128).contiguous(), block, rel_v, "token")
    d = Q.dequant(vc, vz, vs)[:, :, 0].float()                   # (B, Hkv, 128)
    v = v_row.expand(B, Hkv, n_comp + n_res, 128).contiguous().to(dev)
    layer = encode.compress_kv(k[:, :, :n_comp], v[:, :, :n_comp], block=block, bits_k=bits_k, bits_v=bits_v,
                               k_rel=synth.rel_for_bits(bits_k), v_rel=rel_v, k_mode=QuantMode.ChannelQuant)
    flags = ops.new_flags(dev)
    lo = torch.minimum(d, v_row[:, :, 0].float()).repeat_interleave(G, dim=1)
    hi = torch.maximum(d, v_row[:, :, 0].float()).repeat_interleave(G, dim=1)
    tol = TOL * float(v_row.float().abs().max())
    eps = 2.0 ** -8
    lo, hi = torch.minimum(lo * (1 - eps), lo * (1 + eps)), torch.maximum(hi * (1 - eps), hi * (1 + eps))
    out = ops.decode_attention(q, layer, k[:, :, n_comp:].contiguous(), v[:, :, n_comp:].contiguous(), n_res, flags=flags, kv_heads=Hkv).float().cpu()
    assert int(flags.item()) == 0
    assert bool(((out >= lo - tol) & (out <= hi + tol)).all())
    out0 = ops.decode_attention(q, layer, None, None, 0, flags=flags, kv_heads=Hkv).float().cpu()
    assert int(flags.item()) == 0
    dd = d.repeat_interleave(G, dim=1)
    assert bool(((out0 - dd).abs() <= tol + eps * dd.abs()).all())


@pytest.mark.parametrize("cbv", [64, 128])
def test_benchmark_shape_llama8b_vs_oracle(cuda_device, cbv):
    """One sequence of the benchmarked Llama-3.1-8B-shaped layer (8 KV heads x 4 q heads, 8064 compressed +
    128 residual tokens, bf16, 4-bit K per channel / V per token, block 64) against the reference path, with
    the V stream in both token-block layouts: 64 (this library's) and 128 (the only one the reference's
    codec writes, v_encode_cpu.cpp:134-187).  Every warp walks several tiles here, as in the timed launch."""
    err = _run_case(cuda_device, torch.bfloat16, 1, 8, 4, 8064, 128, block=64, cbk=64, cbv=cbv, bits_k=4, bits_v=4,
                    k_mode="channel", seed=1000)
    assert err <= TOL, err


def test_benchmark_shape_qwen8b_long_vs_oracle(cuda_device):
    """One sequence of the long-context layer (32640 compressed + 128 residual tokens, 2-bit K / 4-bit V,
    block 128, bf16) against the reference path."""
    err = _run_case(cuda_device, torch.bfloat16, 1, 8, 4, 32640, 128, block=128, cbk=128, cbv=128, bits_k=2, bits_v=4,
                    k_mode="channel", seed=1001)
    assert err <= TOL, err


@pytest.mark.parametrize("case", [
    # (B, Hkv, G, n_comp, n_res, block, cbv, bits_k, bits_v, k_mode, dtype): 2 to 8 tiles per warp
    (2, 1, 4, 64 * 70, 130, 64, 64, 4, 3, "channel", torch.bfloat16),
    (1, 2, 8, 128 * 45, 16, 64, 128, 3, 4, "token", torch.float16),
    (1, 1, 2, 128 * 100, 191, 128, 128, 2, 2, "channel", torch.float16),
    (3, 1, 4, 64 * 40, 0, 64, 64, 4, 4, "token", torch.bfloat16),
    (1, 4, 1, 128 * 66, 129, 64, 128, 4, 4, "channel", torch.bfloat16),
])
def test_several_tiles_per_warp(cuda_device, case):
    B, Hkv, G, n_comp, n_res, block, cbv, bits_k, bits_v, k_mode, dtype = case
    err = _run_case(cuda_device, dtype, B, Hkv, G, n_comp, n_res, block=block, cbk=block, cbv=cbv, bits_k=bits_k,
                    bits_v=bits_v, k_mode=k_mode, seed=77)
    assert err <= TOL, (case, err)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shift", [4.0, 12.0])
def test_offset_data_large_zero_points(cuda_device, dtype, shift):
    """K and V with a common offset: zero-points of a few tens to ~100 (the in-kernel dequantisation adds
    the zero-point in the element type exactly as the reference does, including its rounding)."""
    dev = cuda_device
    B, Hkv, G, n_comp, n_res = 1, 2, 4, 512, 128
    k, v = synth.synth_kv(B, Hkv, n_comp + n_res, 128, seed=9, dtype=torch.float32, apply_rope=False)
    k, v = (k + shift).to(dtype), (v - shift).to(dtype)
    q = synth.synth_q(B, Hkv * G, 128, seed=9, dtype=dtype)
    layer, kd, vd = layer_from_oracle(k[:, :, :n_comp], v[:, :, :n_comp], block=64, bits_k=4, bits_v=4, k_mode="channel", cbk=64, cbv=64,
                                      rel_k=1 / 14, rel_v=1 / 14, device=dev)
    ref = Q.eager_attention(q, torch.cat([kd, k[:, :, n_comp:]], 2), torch.cat([vd, v[:, :, n_comp:]], 2))[:, 0].float()
    flags = ops.new_flags(dev)
    out = ops.decode_attention(q[:, :, 0].contiguous().to(dev), layer, k[:, :, n_comp:].contiguous().to(dev), v[:, :, n_comp:].contiguous().to(dev),
                               n_res, flags=flags, kv_heads=Hkv)
    torch.cuda.synchronize()
    assert int(flags.item()) == 0
    err = ((out.float().cpu() - ref).abs().max() / ref.abs().max()).item()
    assert err <= TOL, err


def test_zero_point_outside_exact_range_is_flagged(cuda_device):
    """The kernel adds the zero-point to a biased code ((bias + code) + (zero - bias), bias 128 in bf16), which
    equals the reference's code + zero only for -128 <= zero <= 240.  V data with a large common offset has
    zero-points above 240: the launch must say so through PKV_FLAG_ZERO_RANGE instead of returning a slightly
    different answer silently; the same data with the exact (high-precision zero) formula raises no flag."""
    from packkv_b200 import _lib
    dev, dtype = cuda_device, torch.bfloat16
    B, Hkv, G, n_comp = 1, 2, 4, 512
    k, v = synth.synth_kv(B, Hkv, n_comp, 128, seed=9, dtype=torch.float32, apply_rope=False)
    v = (v + 80.0).to(dtype)
    k = k.to(dtype)
    q = synth.synth_q(B, Hkv * G, 128, seed=9, dtype=dtype)[:, :, 0].contiguous().to(dev)
    for hp, want in ((False, _lib.FLAG_ZERO_RANGE), (True, 0)):
        layer, kd, vd = layer_from_oracle(k, v, block=64, bits_k=4, bits_v=4, k_mode="channel", cbk=64, cbv=64,
                                          rel_k=1 / 14, rel_v=1 / 14, device=dev, hp=hp)
        if not hp:
            assert float(layer.v_zero.float().max()) > 240.0      # the case the flag is for
        flags = ops.new_flags(dev)
        out = ops.decode_attention(q, layer, None, None, 0, flags=flags)
        torch.cuda.synchronize()
        assert int(flags.item()) == want
        if hp:
            ref = Q.eager_attention(synth.synth_q(B, Hkv * G, 128, seed=9, dtype=dtype), kd, vd)[:, 0].float()
            assert ((out.float().cpu() - ref).abs().max() / ref.abs().max()).item() <= TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("k_mode", ["channel", "token"])
@pytest.mark.parametrize("bits", [4, 3])
def test_high_precision_zero_point_all_modes(cuda_device, dtype, k_mode, bits):
    """code * scale + min (utils/compute.py:173-176): the product is rounded before the addition, so the
    kernel must not let the pair become one fused multiply-add (that alone moves bf16 outputs by 1e-2)."""
    err = _run_case(cuda_device, dtype, 1, 2, 2, 512, 130, block=64, cbk=64, cbv=64, bits_k=bits, bits_v=bits, k_mode=k_mode, seed=5, hp=True)
    assert err <= TOL, err


def _random_case(it):
    import random
    r = random.Random(1000 + it)
    dtype = r.choice([torch.float16, torch.bfloat16])
    block = r.choice([64, 64, 128])
    cbv = r.choice([64, 128]) if block == 64 else 128
    tile = 128 if (block == 128 or cbv == 128) else 64
    n_comp = tile * r.choice([0, 1, 2, 3, 5, 8, 13, 24])
    n_res = r.choice([0, 1, 15, 16, 17, 128, 130, 160, 191]) if n_comp else r.choice([1, 16, 33, 128, 191])
    return dict(dtype=dtype, B=r.choice([1, 1, 2, 3, 5]), Hkv=r.choice([1, 2, 4, 8]), G=r.choice([1, 2, 3, 4, 5, 7, 8]), n_comp=n_comp,
                n_res=n_res, block=block, cbk=block, cbv=cbv, bits_k=r.choice([2, 3, 4]), bits_v=r.choice([2, 3, 4]),
                k_mode=r.choice(["channel", "token"]), hp=r.random() < 0.25)


@pytest.mark.parametrize("it", range(24))
def test_random_shapes(cuda_device, it):
    """Seeded random draws over batch, heads, group size, lengths (every cluster size and the residual-only
    and compressed-only corners), block sizes, bit widths, K mode and zero-point mode."""
    c = _random_case(it)
    err = _run_case(cuda_device, c["dtype"], c["B"], c["Hkv"], c["G"], c["n_comp"], c["n_res"], block=c["block"], cbk=c["cbk"], cbv=c["cbv"],
                    bits_k=c["bits_k"], bits_v=c["bits_v"], k_mode=c["k_mode"], seed=200 + it, hp=c["hp"])
    assert err <= TOL, (c, err)


# ---- two-launch form: several clusters per (sequence, KV head), state handed over through the scratch ----------
@pytest.mark.parametrize("plan", [(1, 1, 2), (2, 2, 2), (4, 3, 2), (8, 4, 2), (16, 2, 2), (1, 16, 2), (3, 6, 2)])
@pytest.mark.parametrize("k_mode", ["channel", "token"])
def test_split_plans_match_reference(cuda_device, plan, k_mode):
    """(cluster, nsplit) from one cluster in two launches to more warps than tiles, both K modes, V blocks 64 and 128."""
    err = _run_case(cuda_device, torch.bfloat16, 2, 2, 4, 1536, 150, block=64, cbk=64, cbv=128, bits_k=4, bits_v=4, k_mode=k_mode, seed=41, plan=plan,
                    repeats=2)
    assert err <= TOL, err
    err = _run_case(cuda_device, torch.float16, 1, 3, 2, 1024, 129, block=64, cbk=64, cbv=64, bits_k=3, bits_v=2, k_mode=k_mode, seed=42, plan=plan)
    assert err <= TOL, err


def test_split_residual_only_and_high_precision(cuda_device):
    err = _run_case(cuda_device, torch.float16, 2, 2, 4, 0, 191, block=64, cbk=64, cbv=64, bits_k=4, bits_v=4, k_mode="channel", seed=43, plan=(2, 3, 2))
    assert err <= TOL, err
    err = _run_case(cuda_device, torch.bfloat16, 1, 2, 8, 512, 0, block=128, cbk=128, cbv=128, bits_k=2, bits_v=4, k_mode="channel", seed=44, hp=True,
                    plan=(4, 2, 2))
    assert err <= TOL, err


def test_split_chosen_for_one_long_sequence(cuda_device):
    """Batch 1 at a long context: with a scratch the library splits the pairs over several clusters (and says so);
    without one, or with one that is too small, it stays with the single launch; same numbers either way."""
    dev, dtype = cuda_device, torch.bfloat16
    B, Hkv, G, n_comp, n_res = 1, 2, 4, 16384, 130
    k, v = synth.synth_kv(B, Hkv, n_comp + n_res, 128, seed=45, dtype=dtype, apply_rope=True)
    q = synth.synth_q(B, Hkv * G, 128, seed=45, dtype=dtype)
    layer, kd, vd = layer_from_oracle(k[:, :, :n_comp], v[:, :, :n_comp], block=64, bits_k=4, bits_v=4, k_mode="channel", cbk=64, cbv=128,
                                      rel_k=synth.rel_for_bits(4), rel_v=synth.rel_for_bits(4), device=dev)
    ref = Q.eager_attention(q, torch.cat([kd, k[:, :, n_comp:]], 2), torch.cat([vd, v[:, :, n_comp:]], 2))[:, 0].float()
    qd, kr, vr = q[:, :, 0].contiguous().to(dev), k[:, :, n_comp:].contiguous().to(dev), v[:, :, n_comp:].contiguous().to(dev)
    scratch = ops.new_attention_scratch(dev)
    plan = ops.decode_attention(qd, layer, kr, vr, n_res, scratch=scratch, plan_only=True)
    assert plan[2] == 2 and plan[1] > 1, plan
    assert ops.decode_attention(qd, layer, kr, vr, n_res, plan_only=True)[1:] == (1, 1, 0)
    assert ops.decode_attention(qd, layer, kr, vr, n_res, scratch=scratch[:4096], plan_only=True)[1:] == (1, 1, 0)
    flags = ops.new_flags(dev)
    out_split = ops.decode_attention(qd, layer, kr, vr, n_res, flags=flags, scratch=scratch)
    out_one = ops.decode_attention(qd, layer, kr, vr, n_res, flags=flags)
    torch.cuda.synchronize()
    assert int(flags.item()) == 0
    assert _rel_err(out_split.float().cpu(), ref, dtype) <= TOL
    assert _rel_err(out_one.float().cpu(), ref, dtype) <= TOL
    # the same plan on a launch with another batch size gives the same bits for the same sequence
    import dataclasses
    rep = lambda t: t.repeat(3, *([1] * (t.dim() - 1))).contiguous()
    layer3 = dataclasses.replace(layer, **{f: rep(getattr(layer, f)) for f in
                                           ("k_stream", "k_info", "k_bytes", "k_scale", "k_zero", "v_stream", "v_info", "v_bytes", "v_scale", "v_zero")})
    out3 = ops.decode_attention(rep(qd), layer3, rep(kr), rep(vr), n_res, flags=flags, scratch=scratch, plan=plan)
    torch.cuda.synchronize()
    assert int(flags.item()) == 0
    for b in range(3):
        assert torch.equal(out3[b], out_split[0])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("bits", [4, 3, 2])
def test_mixed_pack_widths(cuda_device, dtype, bits):
    """Data in which some channels barely move or hold their value for 32 tokens: packs of 0, 1, 2 bits next to
    full ones in every round (the seeded random data of the other tests has packs of the top two widths only),
    against the same reference, single launch and two launches."""
    dev = cuda_device
    B, Hkv, G, n_comp, n_res = 2, 2, 4, 768, 140
    k, v = synth.synth_kv(B, Hkv, n_comp + n_res, 128, seed=51, dtype=dtype, apply_rope=False)
    q = synth.synth_q(B, Hkv * G, 128, seed=51, dtype=dtype)
    t = torch.arange(n_comp + n_res)
    for x in (k, v):
        xf = x.float()
        xf[..., 1::4] = xf[..., 1::4].mean(dim=2, keepdim=True) + 0.02 * xf[..., 1::4]          # narrow channels
        hold = (t // 32) * 32
        xf[:, :, :, 2::8] = xf[:, :, hold][:, :, :, 2::8] + 0.05 * xf[:, :, :, 2::8]               # channels that hold their value for 32 tokens
        x.copy_(xf.to(dtype))
    for k_mode in ("channel", "token"):
        layer, kd, vd = layer_from_oracle(k[:, :, :n_comp], v[:, :, :n_comp], block=64, bits_k=bits, bits_v=bits, k_mode=k_mode, cbk=64, cbv=128,
                                          rel_k=synth.rel_for_bits(bits), rel_v=synth.rel_for_bits(bits), device=dev)
        # empty, full and in-between widths must be present, or the test does not test what it says
        widths = torch.bincount(layer_pack_widths(k[:, :, :n_comp], bits, k_mode), minlength=5)
        assert widths[0] > 0 and widths[bits] > 0 and int((widths > 0).sum()) >= 3, widths
        ref = Q.eager_attention(q, torch.cat([kd, k[:, :, n_comp:]], 2), torch.cat([vd, v[:, :, n_comp:]], 2))[:, 0].float()
        qd, kr, vr = q[:, :, 0].contiguous().to(dev), k[:, :, n_comp:].contiguous().to(dev), v[:, :, n_comp:].contiguous().to(dev)
        flags = ops.new_flags(dev)
        out = ops.decode_attention(qd, layer, kr, vr, n_res, flags=flags)
        out2 = ops.decode_attention(qd, layer, kr, vr, n_res, flags=flags, scratch=ops.new_attention_scratch(dev), plan=(2, 3, 2))
        torch.cuda.synchronize()
        assert int(flags.item()) == 0
        assert _rel_err(out.float().cpu(), ref, dtype) <= TOL
        assert _rel_err(out2.float().cpu(), ref, dtype) <= TOL


def layer_pack_widths(k, bits, k_mode):
    """Bit widths (0..4) of the K packs (16 tokens of one channel, minimum subtracted), from the oracle's codes."""
    kc, _, _ = Q.quant_ints(k, 64, synth.rel_for_bits(bits), k_mode)
    B, H, nb, blk, D = kc.shape
    c = kc.reshape(B, H, nb * blk // 16, 16, D).int()
    span = c.amax(3) - c.amin(3)
    width = torch.zeros_like(span)
    for b in range(1, 5):
        width[span >= (1 << (b - 1))] = b
    return width.flatten()


@pytest.mark.parametrize("seed", range(12))
def test_random_shapes_single_launch_and_split_agree_with_reference(cuda_device, seed):
    """Seeded random shapes, formats and work splits: the two-launch form with a random (cluster, clusters per pair)
    and the single launch both stay within the bar of the reference path, and the library's own choice with a
    scratch does too."""
    g = torch.Generator().manual_seed(1000 + seed)
    pick = lambda xs: xs[int(torch.randint(len(xs), (1,), generator=g))]
    dtype = pick([torch.float16, torch.bfloat16])
    B, Hkv, G = pick([1, 2, 3]), pick([1, 2, 4]), pick([1, 2, 4, 7, 8])
    cbk, cbv = pick([(64, 64), (64, 128), (128, 128)])
    k_mode = pick(["channel", "token"])
    block = cbk if k_mode == "channel" else 64
    bits_k, bits_v = pick([2, 3, 4]), pick([2, 3, 4])
    tiles = pick([1, 2, 5, 9, 17])
    n_comp = tiles * max(cbk, cbv)
    n_res = pick([0, 1, 17, 128, 191]) if n_comp else 128
    plan = (pick([1, 2, 4, 8, 16]), pick([1, 2, 3, 6]), 2)
    dev = cuda_device
    k, v = synth.synth_kv(B, Hkv, n_comp + n_res, 128, seed=2000 + seed, dtype=dtype, apply_rope=True)
    q = synth.synth_q(B, Hkv * G, 128, seed=2000 + seed, dtype=dtype)
    layer, kd, vd = layer_from_oracle(k[:, :, :n_comp], v[:, :, :n_comp], block=block, bits_k=bits_k, bits_v=bits_v, k_mode=k_mode, cbk=cbk, cbv=cbv,
                                      rel_k=synth.rel_for_bits(bits_k), rel_v=synth.rel_for_bits(bits_v), device=dev)
    ref = Q.eager_attention(q, torch.cat([kd, k[:, :, n_comp:]], 2), torch.cat([vd, v[:, :, n_comp:]], 2))[:, 0].float()
    qd = q[:, :, 0].contiguous().to(dev)
    kr = k[:, :, n_comp:].contiguous().to(dev) if n_res else None
    vr = v[:, :, n_comp:].contiguous().to(dev) if n_res else None
    flags, scratch = ops.new_flags(dev), ops.new_attention_scratch(dev)
    outs = [ops.decode_attention(qd, layer, kr, vr, n_res, flags=flags, kv_heads=Hkv),
            ops.decode_attention(qd, layer, kr, vr, n_res, flags=flags, kv_heads=Hkv, scratch=scratch, plan=plan),
            ops.decode_attention(qd, layer, kr, vr, n_res, flags=flags, kv_heads=Hkv, scratch=scratch)]
    torch.cuda.synchronize()
    assert int(flags.item()) == 0
    for o in outs:
        assert _rel_err(o.float().cpu(), ref, dtype) <= TOL, (seed, plan)


@pytest.mark.parametrize("k_mode", ["channel", "token"])
def test_uneven_ctas_per_pair(cuda_device, k_mode):
    """Two launches of independent CTAs with the pairs getting nsplit or nsplit + 1 of them (the form the library
    chooses when that fills the GPU exactly): forced with small numbers, against the reference; the same plan twice
    gives the same bits, and so does a CUDA-graph-free second call on the same scratch."""
    dev, dtype = cuda_device, torch.bfloat16
    B, Hkv, G, n_comp, n_res = 3, 2, 4, 1920, 150
    k, v = synth.synth_kv(B, Hkv, n_comp + n_res, 128, seed=61, dtype=dtype, apply_rope=True)
    q = synth.synth_q(B, Hkv * G, 128, seed=61, dtype=dtype)
    layer, kd, vd = layer_from_oracle(k[:, :, :n_comp], v[:, :, :n_comp], block=64, bits_k=4, bits_v=3, k_mode=k_mode, cbk=64, cbv=128,
                                      rel_k=synth.rel_for_bits(4), rel_v=synth.rel_for_bits(3), device=dev)
    ref = Q.eager_attention(q, torch.cat([kd, k[:, :, n_comp:]], 2), torch.cat([vd, v[:, :, n_comp:]], 2))[:, 0].float()
    qd, kr, vr = q[:, :, 0].contiguous().to(dev), k[:, :, n_comp:].contiguous().to(dev), v[:, :, n_comp:].contiguous().to(dev)
    flags, scratch = ops.new_flags(dev), ops.new_attention_scratch(dev)
    outs = []
    for plan in [(1, 2, 2, 1), (1, 2, 2, 5), (1, 1, 2, 3), (1, 5, 2, 4), (1, 2, 2, 5)]:
        outs.append(ops.decode_attention(qd, layer, kr, vr, n_res, flags=flags, scratch=scratch, plan=plan))
        torch.cuda.synchronize()
        assert int(flags.item()) == 0
        assert _rel_err(outs[-1].float().cpu(), ref, dtype) <= TOL, plan
        assert ops.decode_attention(qd, layer, kr, vr, n_res, scratch=scratch, plan=plan, plan_only=True) == plan
    assert torch.equal(outs[1], outs[4])
