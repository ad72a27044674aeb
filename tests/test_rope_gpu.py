"""GPU: the cache's rotary embedding (pkv_rope, pkv_append_residual) against the reference's
apply_rotary_pos_emb_single restated on CPU (oracle/quant.py::rope; utils/compute.py:35-43): the
products x * cos and rotate_half(x) * sin are rounded to the element type before they are added, so the
result must be bit-identical."""
import pytest
import torch

from oracle import quant as Q
from packkv_b200 import ops, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [128, 96, 64])
@pytest.mark.parametrize("per_sequence_tables", [False, True])
def test_rope_bit_exact(cuda_device, dtype, D, per_sequence_tables):
    dev = cuda_device
    B, H, T = 3, 5, 37
    g = torch.Generator().manual_seed(D + T)
    x = (torch.randn(B, H, T, D, generator=g) * 3).to(dtype)
    if per_sequence_tables:   # every sequence at its own position, as in a batch of prompts of different lengths
        tabs = [synth.rope_tables(T, D, start=100 * b + 7, dtype=dtype) for b in range(B)]
        cos, sin = torch.cat([t[0] for t in tabs]), torch.cat([t[1] for t in tabs])
    else:
        cos, sin = synth.rope_tables(T, D, start=4000, dtype=dtype)
    want = Q.rope(x, cos.expand(B, T, D), sin.expand(B, T, D))
    got = ops.rope(x.to(dev), cos.to(dev), sin.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))
    # a strided view (heads sliced out of a wider tensor) gives the same result
    wide = torch.zeros(B, H + 2, T, D, dtype=dtype, device=dev)
    wide[:, 1:H + 1] = x.to(dev)
    got2 = ops.rope(wide[:, 1:H + 1], cos.to(dev), sin.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(got2, got)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_append_residual_rotates_k_and_copies_v(cuda_device, dtype):
    dev = cuda_device
    B, H, T, cap, pos = 2, 4, 3, 32, 11
    g = torch.Generator().manual_seed(5)
    k, v = torch.randn(B, H, T, 128, generator=g).to(dtype), torch.randn(B, H, T, 128, generator=g).to(dtype)
    cos, sin = synth.rope_tables(T, 128, start=900, dtype=dtype)
    k_res = torch.full((B, H, cap, 128), 7.0, dtype=dtype, device=dev)
    v_res = torch.full((B, H, cap, 128), -7.0, dtype=dtype, device=dev)
    ops.append_residual(k.to(dev), v.to(dev), k_res, v_res, pos, cos.to(dev), sin.to(dev))
    torch.cuda.synchronize()
    want_k = Q.rope(k, cos.expand(B, T, 128), sin.expand(B, T, 128))
    assert torch.equal(k_res[:, :, pos:pos + T].cpu().view(torch.int16), want_k.view(torch.int16))
    assert torch.equal(v_res[:, :, pos:pos + T].cpu(), v)
    # rows outside [pos, pos + T) are untouched
    assert bool((k_res[:, :, :pos] == 7.0).all()) and bool((k_res[:, :, pos + T:] == 7.0).all())
    assert bool((v_res[:, :, :pos] == -7.0).all()) and bool((v_res[:, :, pos + T:] == -7.0).all())
