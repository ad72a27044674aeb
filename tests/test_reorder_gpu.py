"""GPU: in-block token reordering (median_repacking, utils/compute.py:262-270).

The reference's permutation is only defined up to the order of equal keys (torch's unstable sort),
so the checks are: the sort keys equal torch's lower median bit for bit; the GPU order is the stable
descending order of those keys; the reordered blocks equal the reference's up to the order inside
runs of equal keys (golden fixture from the reference); streams equal the oracle's encoding of the
permuted codes; attention is unchanged."""
import os

import numpy as np
import pytest
import torch

from oracle import codec
from oracle import quant as Q
from packkv_b200 import encode, ops, synth
from packkv_b200.config import QuantMode, RepackMethod

pytestmark = pytest.mark.gpu


def _seq_codes(c5):
    return c5.flatten(2, 3).permute(0, 2, 1, 3).flatten(2, 3).contiguous().to(torch.uint8)


def test_keys_and_order(cuda_device):
    for dtype, B, H, S, block in ((torch.float16, 2, 8, 256, 64), (torch.bfloat16, 1, 2, 384, 128), (torch.float16, 1, 4, 128, 32)):
        _, v = synth.synth_kv(B, H, S, 128, seed=13, dtype=dtype)
        vc, _, _ = Q.quant_ints(v, block, 1 / 14, "token")
        codes = _seq_codes(vc)                                   # (B, S, H*128)
        want_keys = torch.median(codes.float(), dim=2).values.to(torch.uint8)
        order, keys = ops.median_order(codes.to(cuda_device), H, block, want_keys=True)
        torch.cuda.synchronize()
        assert torch.equal(keys.cpu(), want_keys)
        kb = want_keys.view(B, S // block, block).to(torch.int64)
        stable = torch.sort(kb, dim=2, descending=True, stable=True).indices
        assert torch.equal(order.cpu().to(torch.int64), stable)


def test_matches_reference_blocks_up_to_ties(cuda_device, golden_dir):
    g = np.load(os.path.join(golden_dir, "quant_golden.npz"))
    for dname, dtype in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        k = torch.from_numpy(g[f"{dname}_k"]).view(dtype)
        v = torch.from_numpy(g[f"{dname}_v"]).view(dtype)
        kc, _, _ = Q.quant_ints(k, 64, 1 / 14, "channel")
        vc, _, _ = Q.quant_ints(v, 64, 1 / 14, "token")
        B, H = k.shape[0], k.shape[1]
        kcodes, vcodes = _seq_codes(kc).to(cuda_device), _seq_codes(vc).to(cuda_device)
        order = ops.median_order(vcodes, H, 64)
        mine = torch.cat([ops.gather_rows(kcodes, order, 64), ops.gather_rows(vcodes, order, 64)], dim=2)[0].cpu()   # (S, 2F)
        ref = torch.from_numpy(g[f"{dname}_median_blocks"]).reshape(-1, mine.shape[1])                                # reference, B = 1
        F = mine.shape[1] // 2
        key_m = torch.median(mine[:, F:].float(), dim=1).values
        key_r = torch.median(ref[:, F:].float(), dim=1).values
        assert torch.equal(key_m, key_r)                         # same key at every rank
        for blk in range(mine.shape[0] // 64):
            rows_m = sorted(bytes(r.numpy().tobytes()) for r in mine[blk * 64:(blk + 1) * 64])
            rows_r = sorted(bytes(r.numpy().tobytes()) for r in ref[blk * 64:(blk + 1) * 64])
            assert rows_m == rows_r                              # same rows, only tie order may differ


@pytest.mark.parametrize("k_mode", [QuantMode.ChannelQuant, QuantMode.TokenQuant])
def test_reordered_streams_and_attention(cuda_device, k_mode):
    dev, dtype = cuda_device, torch.float16
    B, H, G, S = 2, 2, 4, 512
    k, v = synth.synth_kv(B, H, S, 128, seed=17, dtype=dtype, apply_rope=True)
    q = synth.synth_q(B, H * G, 128, seed=17, dtype=dtype)
    args = dict(block=64, bits_k=4, bits_v=4, k_rel=1 / 14, v_rel=1 / 14, k_mode=k_mode)
    plain = encode.compress_kv(k.to(dev), v.to(dev), **args)
    re = encode.compress_kv(k.to(dev), v.to(dev), repack_method=RepackMethod.MEDIAN, **args)
    torch.cuda.synchronize()
    # streams = oracle encoding of the permuted codes
    mode = "channel" if k_mode == QuantMode.ChannelQuant else "token"
    kc, _, _ = Q.quant_ints(k, 64, 1 / 14, mode)
    vc, _, _ = Q.quant_ints(v, 64, 1 / 14, "token")
    order = re.order.cpu().to(torch.int64)
    R = codec.restated()
    for b in range(B):
        idx = (order[b] + torch.arange(S // 64).unsqueeze(1) * 64).reshape(-1)
        for which, c5, layer_stream, layer_bytes, cb in (("k", kc, re.k_stream, re.k_bytes, 64), ("v", vc, re.v_stream, re.v_bytes, 64)):
            perm_codes = _seq_codes(c5)[b][idx].numpy()
            want, _ = R.encode(which, perm_codes, cb, 4)
            n = int(layer_bytes[b].item())
            assert n == want.size and np.array_equal(layer_stream[b, :n].cpu().numpy(), want)
    # attention is invariant under the in-block permutation
    qd = q[:, :, 0].contiguous().to(dev)
    o1 = ops.decode_attention(qd, plain, None, None, 0).float().cpu()
    o2 = ops.decode_attention(qd, re, None, None, 0).float().cpu()
    assert ((o1 - o2).abs().max() / o1.abs().max()).item() <= 2e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("heads", [2, 8])
def test_order_from_values_equals_order_from_codes(cuda_device, dtype, heads):
    """The single-pass encoder takes its token order from a kernel that never writes codes to memory: it must
    give exactly the order that median_order gives on the quantiser's code matrix (same keys, same stable ties),
    and the per-token parameters of the reordered layer must be the plain layer's, moved with their tokens."""
    dev = cuda_device
    B, S = 3, 320
    k, v = synth.synth_kv(B, heads, S, 128, seed=23, dtype=dtype, device=dev, apply_rope=True)
    vq = ops.quantize(v, 64, 1 / 14, ops.K_TOKEN, bits=4)
    want = ops.median_order(vq.codes, heads, 64)
    got = ops.value_median_order(v, 64, 1 / 14)
    assert torch.equal(got, want)
    args = dict(block=64, bits_k=4, bits_v=4, k_rel=1 / 14, v_rel=1 / 14, k_mode=QuantMode.TokenQuant)
    plain = encode.compress_kv(k, v, **args)
    re = encode.compress_kv(k, v, repack_method=RepackMethod.MEDIAN, **args)
    assert torch.equal(re.order, want)
    idx = (want.to(torch.int64) + torch.arange(S // 64, device=dev).view(1, -1, 1) * 64).reshape(B, S)
    for name in ("v_scale", "v_zero", "k_scale", "k_zero"):
        assert torch.equal(getattr(re, name)[:, :S], torch.gather(getattr(plain, name)[:, :S], 1, idx)), name


def _feature_blocks(kcodes, vcodes, block):
    """(S, hidden) K and V codes of one sequence -> (n_blocks, block, 2*hidden) like compute.py:336-338."""
    S = kcodes.shape[0]
    return torch.cat([kcodes, vcodes], dim=1).view(S // block, block, -1)


def test_greedy_order_matches_reference_golden(cuda_device, golden_dir):
    """greedy_repacking (utils/compute.py:210-260): identical permuted blocks on the golden inputs."""
    g = np.load(os.path.join(golden_dir, "quant_golden.npz"))
    for dname, dtype in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        k = torch.from_numpy(g[f"{dname}_k"]).view(dtype)
        v = torch.from_numpy(g[f"{dname}_v"]).view(dtype)
        kc, _, _ = Q.quant_ints(k, 64, 1 / 14, "channel")
        vc, _, _ = Q.quant_ints(v, 64, 1 / 14, "token")
        H = k.shape[1]
        kcodes, vcodes = _seq_codes(kc).to(cuda_device), _seq_codes(vc).to(cuda_device)
        order = ops.greedy_order(kcodes, vcodes, H, 64, 16)
        mine = torch.cat([ops.gather_rows(kcodes, order, 64), ops.gather_rows(vcodes, order, 64)], dim=2)[0].cpu()
        ref = torch.from_numpy(g[f"{dname}_greedy_blocks"]).reshape(-1, mine.shape[1])
        assert torch.equal(mine, ref)
        # the size model before and after, K and V halves (repack_and_encode, compute.py:328-357)
        pre = (ops.size_model(kcodes, 16), ops.size_model(vcodes, 16))
        aft = (ops.size_model(ops.gather_rows(kcodes, order, 64), 16), ops.size_model(ops.gather_rows(vcodes, order, 64), 16))
        assert [pre[0], pre[1], aft[0], aft[1]] == list(g[f"{dname}_greedy_sizes"])


@pytest.mark.parametrize("shape", [(2, 2, 256, 64, 16), (1, 8, 128, 64, 16), (1, 2, 256, 128, 16), (2, 1, 128, 32, 8)])
def test_greedy_order_matches_oracle(cuda_device, shape):
    B, H, S, block, pack = shape
    k, v = synth.synth_kv(B, H, S, 128, seed=23, dtype=torch.float16, apply_rope=True)
    kc, _, _ = Q.quant_ints(k, block, 1 / 14, "channel")
    vc, _, _ = Q.quant_ints(v, block, 1 / 6, "token")           # 3-bit V: more ties
    kcodes, vcodes = _seq_codes(kc), _seq_codes(vc)
    order = ops.greedy_order(kcodes.to(cuda_device), vcodes.to(cuda_device), H, block, pack).cpu().to(torch.int64)
    for b in range(B):
        want = Q.greedy_order(_feature_blocks(kcodes[b], vcodes[b], block), pack)
        assert torch.equal(order[b], want)
    for b in range(B):                                           # size model of each tensor against the oracle's
        blocks = _feature_blocks(kcodes[b:b + 1].reshape(S, -1), vcodes[b:b + 1].reshape(S, -1), block)
        want_k, want_v = Q.size_model(blocks, pack)
        assert ops.size_model(kcodes[b:b + 1].to(cuda_device), pack) == want_k
        assert ops.size_model(vcodes[b:b + 1].to(cuda_device), pack) == want_v


def test_greedy_streams_and_attention(cuda_device):
    dev, dtype = cuda_device, torch.float16
    B, H, G, S = 2, 2, 4, 256
    k, v = synth.synth_kv(B, H, S, 128, seed=29, dtype=dtype, apply_rope=True)
    q = synth.synth_q(B, H * G, 128, seed=29, dtype=dtype)
    args = dict(block=64, bits_k=4, bits_v=4, k_rel=1 / 14, v_rel=1 / 14, k_mode=QuantMode.ChannelQuant)
    plain = encode.compress_kv(k.to(dev), v.to(dev), **args)
    re = encode.compress_kv(k.to(dev), v.to(dev), repack_method=RepackMethod.GREEDY, **args)
    torch.cuda.synchronize()
    kc, _, _ = Q.quant_ints(k, 64, 1 / 14, "channel")
    vc, _, _ = Q.quant_ints(v, 64, 1 / 14, "token")
    R = codec.restated()
    for b in range(B):
        want_order = Q.greedy_order(_feature_blocks(_seq_codes(kc)[b], _seq_codes(vc)[b], 64), 16)
        assert torch.equal(re.order[b].cpu().to(torch.int64), want_order)
        idx = (want_order + torch.arange(S // 64).unsqueeze(1) * 64).reshape(-1)
        for which, c5, layer_stream, layer_bytes in (("k", kc, re.k_stream, re.k_bytes), ("v", vc, re.v_stream, re.v_bytes)):
            want, _ = R.encode(which, _seq_codes(c5)[b][idx].numpy(), 64, 4)
            n = int(layer_bytes[b].item())
            assert n == want.size and np.array_equal(layer_stream[b, :n].cpu().numpy(), want)
    assert int(re.k_bytes.sum()) + int(re.v_bytes.sum()) < int(plain.k_bytes.sum()) + int(plain.v_bytes.sum())
    qd = q[:, :, 0].contiguous().to(dev)
    o1 = ops.decode_attention(qd, plain, None, None, 0).float().cpu()
    o2 = ops.decode_attention(qd, re, None, None, 0).float().cpu()
    assert ((o1 - o2).abs().max() / o1.abs().max()).item() <= 2e-3
