"""GPU: the reference's packkv_cuda entry points, driven the way the reference's own harness
drives them (evaluation/evaluation.py:398-524 for K, :587-715 for V): quantise, flatten to
(ctx, hidden) uint8, encode into caller-allocated CPU buffers, decode and compare, then the
two-step matvec + epilogue against a dense fp32 product."""
import numpy as np
import pytest
import torch

import packkv_cuda
from oracle import codec
from oracle import quant as Q
from packkv_b200 import synth

pytestmark = pytest.mark.gpu
U32 = getattr(torch, "uint32", torch.int32)


def _pipeline(x, mode, rel):
    c, z, s = Q.quant_ints(x, 64, rel, mode)
    deq = ((c + z) * s).flatten(2, 3)
    mat = c.flatten(2, 3).permute(2, 0, 1, 3).flatten(1, 3).contiguous().to(torch.uint8)
    return mat, z.flatten(), s.flatten(), deq


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_k_path_like_the_reference_harness(cuda_device, dtype):
    k, _ = synth.synth_kv(1, 8, 1024, 128, seed=0, dtype=dtype)
    block, zero, scale, k_deq = _pipeline(k, "token", 0.1)
    ctx_len, hidden = block.shape
    assert int(np.ceil(np.log2(block.unique().numel()))) == 4          # evaluation.py:416-417
    info = torch.zeros((ctx_len // 64) * (hidden // 128), 2, dtype=U32)
    compressed = torch.zeros_like(block)
    size = packkv_cuda.k_encode_cpu(block, compressed, info, ctx_len, hidden, 64, 128, 4)
    ref_stream, ref_info = codec.restated().encode("k", block.numpy(), 64, 4)
    assert size == ref_stream.size
    assert np.array_equal(compressed.view(-1)[:size].numpy(), ref_stream)
    assert np.array_equal(info.view(torch.int32).numpy().view(np.uint32), ref_info)
    back = torch.zeros_like(block)
    packkv_cuda.k_decode_cpu(compressed, info, back, ctx_len, hidden, 64, 128, 4)
    assert (block == back).all()                                        # evaluation.py:456

    heads = hidden // 128
    torch.manual_seed(1)
    q = torch.randn(heads, 128, dtype=dtype).to(cuda_device)
    qr = q.view(heads, 32, 4)
    q_t = torch.cat([qr[:, :, :2].contiguous().view(heads, -1), qr[:, :, 2:].contiguous().view(heads, -1)], dim=1)
    t = torch.zeros(heads, ctx_len, dtype=dtype, device=cuda_device)
    ms = packkv_cuda.kq_mat_vec_mul(compressed.to(cuda_device), info.to(cuda_device), q_t.contiguous(), t, ctx_len, hidden, 64, 128, 4)
    assert ms >= 0
    codes = block.to(cuda_device).view(ctx_len, heads, 128).float()
    want_t = torch.einsum("nhd,hd->hn", codes, q.float())
    assert ((t.float() - want_t).abs().max() / want_t.abs().max()).item() < (2e-3 if dtype == torch.float16 else 1e-2)
    our = torch.empty_like(t)
    packkv_cuda.fused_kq(our, q, zero.to(cuda_device), scale.to(cuda_device), t)
    target = (k_deq.squeeze(0).to(cuda_device).float() @ q.float().unsqueeze(2)).squeeze()
    err = ((target - our.float()).abs() / target.abs().max()).max().item() * 100
    # t is stored in the element type between the two calls (the reference's API), so bf16 loses
    # bits to the cancellation between sum(q)*zero and t; the reference accepts 10 % (evaluation.py:514-519)
    assert err < (1.0 if dtype == torch.float16 else 10.0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_v_path_like_the_reference_harness(cuda_device, dtype):
    _, v = synth.synth_kv(1, 8, 1024, 128, seed=0, dtype=dtype)
    block, zero, scale, v_deq = _pipeline(v, "token", 0.2)
    ctx_len, hidden = block.shape
    bits = int(np.ceil(np.log2(block.unique().numel())))
    assert bits == 3
    info = torch.zeros((ctx_len // 128) * (hidden // 64), 2, dtype=U32)
    compressed = torch.zeros_like(block)
    size = packkv_cuda.v_encode_cpu(block, compressed, info, ctx_len, hidden, 128, 64, bits)
    ref_stream, ref_info = codec.restated().encode("v", block.numpy(), 128, bits)
    assert size == ref_stream.size and np.array_equal(compressed.view(-1)[:size].numpy(), ref_stream)
    back = torch.zeros_like(block)
    packkv_cuda.v_decode_cpu(compressed, info, back, ctx_len, hidden, 128, 64, bits)
    assert (block == back).all()                                        # evaluation.py:644

    heads = hidden // 128
    torch.manual_seed(2)
    w = torch.randn(heads, ctx_len, dtype=dtype).to(cuda_device).pow(2).softmax(dim=1)
    term1 = torch.zeros(heads, 128, dtype=torch.float32, device=cuda_device)
    w_prime = (w * scale.to(cuda_device).unsqueeze(0)).contiguous()
    packkv_cuda.wv_mat_vec_mul(compressed.to(cuda_device), info.to(cuda_device), w_prime, term1, ctx_len, hidden, 128, 64, bits)
    codes = block.to(cuda_device).view(ctx_len, heads, 128).float()
    want = torch.einsum("hn,nhd->hd", w_prime.float(), codes)
    assert ((term1 - want).abs().max() / want.abs().max()).item() < 1e-4
    # accumulate semantics: a second call doubles the result
    packkv_cuda.wv_mat_vec_mul(compressed.to(cuda_device), info.to(cuda_device), w_prime, term1, ctx_len, hidden, 128, 64, bits)
    assert ((term1 - 2 * want).abs().max() / want.abs().max()).item() < 2e-4
    term1 = (term1 / 2).to(dtype)
    our = torch.empty_like(term1)
    packkv_cuda.fused_wv(our, w, zero.to(cuda_device), scale.to(cuda_device), term1)
    target = (w.float().unsqueeze(1) @ v_deq.squeeze(0).to(cuda_device).float()).squeeze()
    err = ((target - our.float()).abs() / target.abs().max()).max().item() * 100
    assert err < (1.0 if dtype == torch.float16 else 3.0)    # the reference accepts 6 % (evaluation.py:704-709)


def test_error_behaviour(cuda_device):
    block = torch.zeros(64, 128, dtype=torch.uint8)
    info = torch.zeros(1, 2, dtype=U32)
    buf = torch.zeros_like(block)
    with pytest.raises(RuntimeError, match="not supported"):     # the reference's dispatch failure
        packkv_cuda.k_encode_cpu(block, buf, info, 64, 128, 64, 128, 1)
    with pytest.raises(ValueError):                                # the reference aborts the process here
        packkv_cuda.k_encode_cpu(block, buf, info, 64, 128, 64, 64, 4)
    with pytest.raises(ValueError):
        packkv_cuda.k_encode_cpu(block, buf, torch.zeros(2, 2, dtype=U32), 64, 128, 64, 128, 4)
    with pytest.raises(ValueError):
        packkv_cuda.k_encode_cpu(block.float(), buf, info, 64, 128, 64, 128, 4)
    # CUDA tensors are accepted directly
    size = packkv_cuda.k_encode_cpu(block.to(cuda_device), buf.to(cuda_device), info.to(cuda_device), 64, 128, 64, 128, 4)
    assert size == 8 + 4 * (64 + 48)
