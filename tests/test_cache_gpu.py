"""GPU: the cache class and its append path against the reference's cache state machine restated
on CPU (oracle/quant.py CacheLayerOracle: RoPE -> cut whole blocks -> quantise -> dequantise ->
cat).  Dense views must be bit-identical; fused attention within 2e-3."""
import pytest
import torch

from oracle import quant as Q
from packkv_b200 import cache as C
from packkv_b200 import synth
from packkv_b200.config import PackKVCacheConfig, QuantMethod, RepackMethod

pytestmark = pytest.mark.gpu


def _cfg(method, k_rel=1 / 14, v_rel=1 / 14, hp=False, enable=True, repack=RepackMethod.NONE):
    return PackKVCacheConfig("synthetic", method, repack, hp, 64, 192, 16, k_rel, v_rel, enable_quant=enable)


def _modes(method):
    return {QuantMethod.KIVI: ("channel", "token"), QuantMethod.PackKV: ("token", "token")}[method]


@pytest.mark.parametrize("method,repack", [(QuantMethod.KIVI, RepackMethod.NONE), (QuantMethod.PackKV, RepackMethod.NONE),
                                           (QuantMethod.KIVI, RepackMethod.MEDIAN), (QuantMethod.PackKV, RepackMethod.MEDIAN)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_prefill_then_decode_matches_reference_cache(cuda_device, method, repack, dtype):
    dev = cuda_device
    B, H, G, S0, steps = 2, 2, 4, 333, 140
    cfg = _cfg(method, repack=repack)
    C.PackKVCacheConfigStatic.config = cfg
    try:
        cache = C.PackKVCache(B, H * G, 128, 1, materialize=True)
        km, vm = _modes(method)
        oracle = Q.CacheLayerOracle(64, 192, cfg.k_quant_scale_rel, cfg.v_quant_scale_rel, km, vm)
        k, v = synth.synth_kv(B, H, S0 + steps, 128, seed=31, dtype=dtype)
        cos, sin = synth.rope_tables(S0 + steps, 128, dtype=dtype)
        # prefill
        Ko, Vo = oracle.update(k[:, :, :S0], v[:, :, :S0], cos[:, :S0], sin[:, :S0])
        Kg, Vg = cache.update(k[:, :, :S0].to(dev), v[:, :, :S0].to(dev), 0, {"cos": cos[:, :S0].to(dev), "sin": sin[:, :S0].to(dev)})
        assert torch.equal(Kg.cpu(), Ko) and torch.equal(Vg.cpu(), Vo)
        assert cache.get_seq_length(0) == oracle.seq_length() == S0
        # decode: one token at a time; the residual stays within [128, 191]
        for t in range(S0, S0 + steps):
            Ko, Vo = oracle.update(k[:, :, t:t + 1], v[:, :, t:t + 1], cos[:, t:t + 1], sin[:, t:t + 1])
            Kg, Vg = cache.update(k[:, :, t:t + 1].to(dev), v[:, :, t:t + 1].to(dev), 0,
                                  {"cos": cos[:, t:t + 1].to(dev), "sin": sin[:, t:t + 1].to(dev)})
            assert 128 <= cache._layers[0].n_res <= 191
            assert cache.get_seq_length(0) == t + 1
            if (t - S0) % 16 == 0 or t == S0 + steps - 1:
                assert torch.equal(Kg.cpu(), Ko), t
                assert torch.equal(Vg.cpu(), Vo), t
                q = synth.synth_q(B, H * G, 128, seed=t, dtype=dtype)
                ref = Q.eager_attention(q, Ko, Vo).float()
                out = cache.attend(q.to(dev), 0).float().cpu()
                assert ((out - ref).abs().max() / ref.abs().max()).item() <= 2e-3, t
        cache.check_flags()
        assert cache.compressed_bytes() > 0
    finally:
        C.PackKVCacheConfigStatic.config = None


@pytest.mark.parametrize("method", [QuantMethod.KIVI, QuantMethod.PackKV])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_high_precision_zero_and_three_bit_cache(cuda_device, method, dtype):
    """high_precision_zero_point=True (zero = block minimum, utils/compute.py:97-101) with 3-bit scales:
    dense views bit-identical to the reference cache, fused attention within 2e-3."""
    dev = cuda_device
    B, H, G, S0, steps = 1, 2, 4, 260, 70
    cfg = _cfg(method, k_rel=1 / 6, v_rel=1 / 6, hp=True)
    C.PackKVCacheConfigStatic.config = cfg
    try:
        cache = C.PackKVCache(B, H * G, 128, 1, materialize=True)
        km, vm = _modes(method)
        oracle = Q.CacheLayerOracle(64, 192, 1 / 6, 1 / 6, km, vm, high_precision_zero=True)
        k, v = synth.synth_kv(B, H, S0 + steps, 128, seed=37, dtype=dtype)
        cos, sin = synth.rope_tables(S0 + steps, 128, dtype=dtype)
        Ko, Vo = oracle.update(k[:, :, :S0], v[:, :, :S0], cos[:, :S0], sin[:, :S0])
        Kg, Vg = cache.update(k[:, :, :S0].to(dev), v[:, :, :S0].to(dev), 0, {"cos": cos[:, :S0].to(dev), "sin": sin[:, :S0].to(dev)})
        assert torch.equal(Kg.cpu(), Ko) and torch.equal(Vg.cpu(), Vo)
        for t in range(S0, S0 + steps):
            Ko, Vo = oracle.update(k[:, :, t:t + 1], v[:, :, t:t + 1], cos[:, t:t + 1], sin[:, t:t + 1])
            Kg, Vg = cache.update(k[:, :, t:t + 1].to(dev), v[:, :, t:t + 1].to(dev), 0,
                                  {"cos": cos[:, t:t + 1].to(dev), "sin": sin[:, t:t + 1].to(dev)})
        assert torch.equal(Kg.cpu(), Ko) and torch.equal(Vg.cpu(), Vo)
        q = synth.synth_q(B, H * G, 128, seed=3, dtype=dtype)
        ref = Q.eager_attention(q, Ko, Vo).float()
        out = cache.attend(q.to(dev), 0).float().cpu()
        assert ((out - ref).abs().max() / ref.abs().max()).item() <= 2e-3
        cache.check_flags()
    finally:
        C.PackKVCacheConfigStatic.config = None


@pytest.mark.parametrize("method", [QuantMethod.KIVI, QuantMethod.PackKV])
@pytest.mark.parametrize("head_dim", [96, 64])
def test_head_dim_below_128_matches_reference_cache(cuda_device, method, head_dim):
    """Phi-3-style heads (head_dim 96, MHA): the cache stores them in 128-channel blocks whose tail repeats the
    first channels, which leaves every real channel's codes and parameters those of the reference's cache run on
    head_dim-wide tensors (models/phi.py:744-747 creates the cache with hidden_size // num_attention_heads).
    Dense views bit-identical, fused attention within 2e-3, prefill + decode across a block boundary."""
    dev, dtype = cuda_device, torch.bfloat16
    B, H, G, S0, steps, D = 2, 4, 1, 270, 70, head_dim
    cfg = _cfg(method)
    C.PackKVCacheConfigStatic.config = cfg
    try:
        cache = C.PackKVCache(B, H * G, D, 1, materialize=True)
        km, vm = _modes(method)
        oracle = Q.CacheLayerOracle(64, 192, cfg.k_quant_scale_rel, cfg.v_quant_scale_rel, km, vm)
        k, v = synth.synth_kv(B, H, S0 + steps, D, seed=41, dtype=dtype)
        cos, sin = synth.rope_tables(S0 + steps, D, dtype=dtype)
        Ko, Vo = oracle.update(k[:, :, :S0], v[:, :, :S0], cos[:, :S0], sin[:, :S0])
        Kg, Vg = cache.update(k[:, :, :S0].to(dev), v[:, :, :S0].to(dev), 0, {"cos": cos[:, :S0].to(dev), "sin": sin[:, :S0].to(dev)})
        assert Kg.shape[-1] == D and torch.equal(Kg.cpu(), Ko) and torch.equal(Vg.cpu(), Vo)
        for t in range(S0, S0 + steps):
            Ko, Vo = oracle.update(k[:, :, t:t + 1], v[:, :, t:t + 1], cos[:, t:t + 1], sin[:, t:t + 1])
            Kg, Vg = cache.update(k[:, :, t:t + 1].to(dev), v[:, :, t:t + 1].to(dev), 0,
                                  {"cos": cos[:, t:t + 1].to(dev), "sin": sin[:, t:t + 1].to(dev)})
        assert torch.equal(Kg.cpu(), Ko) and torch.equal(Vg.cpu(), Vo)
        q = synth.synth_q(B, H * G, D, seed=5, dtype=dtype)
        ref = Q.eager_attention(q, Ko, Vo).float()                  # scaling head_dim ** -0.5
        out = cache.attend(q.to(dev), 0).float().cpu()
        assert out.shape == ref.shape
        assert ((out - ref).abs().max() / ref.abs().max()).item() <= 2e-3
        cache.check_flags()
    finally:
        C.PackKVCacheConfigStatic.config = None


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decode_step_append_inside_the_attention_launch(cuda_device, dtype):
    """A decode step without materialised K/V: update() only records the new token, attend() lets the attention
    launch rotate K, write both rows into the residual and attend over them.  The residual rows must equal the
    ones pkv_append_residual writes (bit for bit, same RoPE arithmetic), the attention output the reference's
    within 2e-3, and an update() that is not followed by attend() must still land in the residual."""
    dev = cuda_device
    B, H, G, S0, steps = 2, 2, 4, 300, 40
    cfg = _cfg(QuantMethod.KIVI)
    C.PackKVCacheConfigStatic.config = cfg
    try:
        fused, plain = C.PackKVCache(B, H * G, 128, 1), C.PackKVCache(B, H * G, 128, 1, materialize=True)
        oracle = Q.CacheLayerOracle(64, 192, cfg.k_quant_scale_rel, cfg.v_quant_scale_rel, "channel", "token")
        k, v = synth.synth_kv(B, H, S0 + steps, 128, seed=51, dtype=dtype)
        cos, sin = synth.rope_tables(S0 + steps, 128, dtype=dtype)
        kw = lambda a, b: {"cos": cos[:, a:b].to(dev), "sin": sin[:, a:b].to(dev)}
        Ko, Vo = oracle.update(k[:, :, :S0], v[:, :, :S0], cos[:, :S0], sin[:, :S0])
        for c in (fused, plain):
            c.update(k[:, :, :S0].to(dev), v[:, :, :S0].to(dev), 0, kw(0, S0))
        for t in range(S0, S0 + steps):
            Ko, Vo = oracle.update(k[:, :, t:t + 1], v[:, :, t:t + 1], cos[:, t:t + 1], sin[:, t:t + 1])
            n_comp_before = fused._layers[0].n_comp
            for c in (fused, plain):
                c.update(k[:, :, t:t + 1].to(dev), v[:, :, t:t + 1].to(dev), 0, kw(t, t + 1))
            if t % 3 == 0:
                continue                                             # no attend(): the next update() must flush the token
            # a step that moved a block out of the residual went through the ordinary path; every other step defers
            assert (fused._layers[0].pending is not None) == (fused._layers[0].n_comp == n_comp_before)
            q = synth.synth_q(B, H * G, 128, seed=t, dtype=dtype)
            out = fused.attend(q.to(dev), 0).float().cpu()
            assert fused._layers[0].pending is None
            ref = Q.eager_attention(q, Ko, Vo).float()
            assert ((out - ref).abs().max() / ref.abs().max()).item() <= 2e-3, t
            Lf, Lp = fused._layers[0], plain._layers[0]
            assert Lf.n_res == Lp.n_res
            assert torch.equal(Lf.k_res[:, :, : Lf.n_res], Lp.k_res[:, :, : Lp.n_res]), t
            assert torch.equal(Lf.v_res[:, :, : Lf.n_res], Lp.v_res[:, :, : Lp.n_res]), t
        Kd, Vd = fused.dense(0)
        assert torch.equal(Kd.cpu(), Ko) and torch.equal(Vd.cpu(), Vo)
        fused.check_flags()
    finally:
        C.PackKVCacheConfigStatic.config = None


def test_append_streams_equal_one_shot_encode(cuda_device):
    """Blocks appended one at a time give the same bytes as encoding the history in one call."""
    from packkv_b200 import encode, ops
    from packkv_b200.config import QuantMode
    dev = cuda_device
    C.PackKVCacheConfigStatic.config = _cfg(QuantMethod.KIVI)
    try:
        B, H, S = 2, 2, 64 * 9
        cache = C.PackKVCache(B, H, 128, 1)
        k, v = synth.synth_kv(B, H, S, 128, seed=5, dtype=torch.float16)
        cos, sin = synth.rope_tables(S, 128, dtype=torch.float16)
        cos1, sin1 = torch.ones_like(cos), torch.zeros_like(sin)      # identity rotation keeps K as is
        cache.update(k[:, :, :200].to(dev), v[:, :, :200].to(dev), 0, {"cos": cos1[:, :200].to(dev), "sin": sin1[:, :200].to(dev)})
        for t in range(200, S):
            cache.update(k[:, :, t:t + 1].to(dev), v[:, :, t:t + 1].to(dev), 0, {"cos": cos1[:, t:t + 1].to(dev), "sin": sin1[:, t:t + 1].to(dev)})
        L = cache._layers[0]
        n = L.n_comp
        assert n == S - 128 - S % 64 and n > 0
        one = encode.compress_kv(k[:, :, :n].to(dev), v[:, :, :n].to(dev), block=64, bits_k=4, bits_v=4, k_rel=1 / 14, v_rel=1 / 14,
                                 k_mode=QuantMode.ChannelQuant)
        torch.cuda.synchronize()
        for b in range(B):
            nk, nv = int(one.k_bytes[b].item()), int(one.v_bytes[b].item())
            assert int(L.comp.k_bytes[b].item()) == nk and int(L.comp.v_bytes[b].item()) == nv
            assert torch.equal(L.comp.k_stream[b, :nk], one.k_stream[b, :nk])
            assert torch.equal(L.comp.v_stream[b, :nv], one.v_stream[b, :nv])
        nkb, nvb = one.k_info.shape[1], one.v_info.shape[1]
        assert torch.equal(L.comp.k_info[:, : (n // 64) * H], one.k_info[:, : (n // 64) * H])
        assert torch.equal(L.comp.v_info[:, : (n // 64) * 2 * H], one.v_info[:, : (n // 64) * 2 * H])
    finally:
        C.PackKVCacheConfigStatic.config = None


def test_config_contract_and_disabled_quant(cuda_device):
    dev = cuda_device
    C.PackKVCacheConfigStatic.config = None
    cache = C.PackKVCache(1, 8, 128, 2)
    k, v = synth.synth_kv(1, 2, 10, 128, seed=1, dtype=torch.float16)
    cos, sin = synth.rope_tables(10, 128, dtype=torch.float16)
    kw = {"cos": cos.to(dev), "sin": sin.to(dev)}
    with pytest.raises(ValueError):                     # packkv_quant.py:54-55
        cache.update(k.to(dev), v.to(dev), 0, kw)
    with pytest.raises(ValueError):
        cache.get_seq_length(0)
    C.PackKVCacheConfigStatic.config = _cfg(QuantMethod.KIVI, enable=False)
    try:
        K, V = cache.update(k.to(dev), v.to(dev), 1, kw)
        assert torch.equal(K.cpu(), Q.rope(k, cos, sin)) and torch.equal(V.cpu(), v)
        K, V = cache.update(k[:, :, :1].to(dev), v[:, :, :1].to(dev), 1, {"cos": cos[:, :1].to(dev), "sin": sin[:, :1].to(dev)})
        assert K.shape[2] == 11 and cache.get_seq_length(1) == 11 and cache.get_seq_length(0) == 0
    finally:
        C.PackKVCacheConfigStatic.config = None
    cfg = _cfg(QuantMethod.KIVI, k_rel=0.1, v_rel=0.2)
    assert PackKVCacheConfig.from_str(str(cfg)) == cfg and hash(PackKVCacheConfig.from_str(str(cfg))) == hash(cfg)
    assert C.bits_for_rel(0.1) == 4 and C.bits_for_rel(0.2) == 3 and C.bits_for_rel(1 / 14) == 4 and C.bits_for_rel(0.5) == 2
