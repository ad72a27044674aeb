"""Blob format of the serialised compressed cache (CPU: bytes only) and, on the GPU, that a
restored layer / cache decodes to exactly the same attention output and keeps appending."""
import pytest
import torch

from packkv_b200 import ops, serialize


def _fake_layer(order=False):
    g = torch.Generator().manual_seed(5)
    B, H, n, cb = 2, 2, 128, 64
    r = lambda *s: torch.randint(0, 255, s, dtype=torch.uint8, generator=g)
    k_bytes = torch.tensor([900, 1000], dtype=torch.int32)
    return ops.CompressedLayer(
        k_stream=r(B, 4096), k_info=torch.randint(0, 1000, (B, 8, 2), dtype=torch.int32, generator=g), k_bytes=k_bytes,
        k_scale=torch.randn(B, H, 4, 128, generator=g).half(), k_zero=torch.randn(B, H, 4, 128, generator=g).half(),
        v_stream=r(B, 4096), v_info=torch.randint(0, 1000, (B, 16, 2), dtype=torch.int32, generator=g), v_bytes=k_bytes + 7,
        v_scale=torch.randn(B, 256, generator=g).half(), v_zero=torch.randn(B, 256, generator=g).half(),
        n_comp=n, kv_heads=H, cbk=cb, cbv=cb, bits_k=4, bits_v=3, k_mode=ops.K_CHANNEL,
        order=torch.randint(0, 64, (B, 2, 64), dtype=torch.uint8, generator=g) if order else None)


@pytest.mark.parametrize("order", [False, True])
def test_layer_blob_roundtrip_cpu(order):
    L = _fake_layer(order)
    blob = serialize.dumps_layer(L)
    assert blob[:4] == b"PKVC" and len(blob) % 16 == 0
    R = serialize.loads_layer(blob, device="cpu")
    assert (R.n_comp, R.kv_heads, R.cbk, R.cbv, R.bits_k, R.bits_v, R.k_mode) == (128, 2, 64, 64, 4, 3, ops.K_CHANNEL)
    assert torch.equal(R.k_stream[:, :1008], L.k_stream[:, :1008]) and R.k_stream.shape[1] == 1008 + 32
    assert torch.equal(R.v_stream[:, :1008], L.v_stream[:, :1008])
    assert torch.equal(R.k_info, L.k_info[:, :4]) and torch.equal(R.v_info, L.v_info[:, :8])
    assert torch.equal(R.k_scale, L.k_scale[:, :, :2]) and torch.equal(R.v_zero, L.v_zero[:, :128])
    assert (R.order is None) == (not order) and (not order or torch.equal(R.order, L.order))


def test_rejects_garbage():
    with pytest.raises(ValueError):
        serialize.loads_layer(b"nope" + b"\0" * 40, device="cpu")
    blob = serialize.dumps_layer(_fake_layer())
    with pytest.raises(ValueError):
        serialize.loads_layer(blob[: len(blob) // 2], device="cpu")
    with pytest.raises(ValueError):
        serialize.loads_cache(blob, device="cpu")


def test_rejects_metadata_that_disagrees_with_the_arrays():
    """The attention kernel indexes the block tables and parameter arrays from n_comp, kv_heads and the block
    sizes: a layer (restored from a blob or built by a caller) that claims more tokens or heads than its arrays
    hold, or another batch than q, must raise on the host and never reach the device."""
    for field, value in (("cbk", 32), ("bits_v", 7), ("k_mode", 5)):
        L = _fake_layer()
        setattr(L, field, value)
        with pytest.raises((ValueError, RuntimeError)):
            serialize.loads_layer(serialize.dumps_layer(L), device="cpu")
    for field, value in (("n_comp", 4096), ("kv_heads", 16)):
        L = _fake_layer()
        setattr(L, field, value)
        with pytest.raises(ValueError):
            ops._check_layer_shapes(L, 2)
    with pytest.raises(ValueError):
        ops._check_layer_shapes(_fake_layer(), 3)          # q with another batch size
    L = _fake_layer()
    L.v_info = L.v_info[:, :3]
    with pytest.raises(ValueError):
        ops._check_layer_shapes(L, 2)


@pytest.mark.gpu
def test_restored_layer_and_cache_decode_identically(cuda_device):
    from packkv_b200 import encode, synth
    from packkv_b200.cache import PackKVCache, PackKVCacheConfigStatic
    from packkv_b200.config import PackKVCacheConfig, QuantMethod, QuantMode, RepackMethod
    dev, dtype = cuda_device, torch.bfloat16
    B, H, G, S = 2, 2, 4, 512
    k, v = synth.synth_kv(B, H, S + 80, 128, seed=31, dtype=dtype, apply_rope=False)
    q = synth.synth_q(B, H * G, 128, seed=31, dtype=dtype)[:, :, 0].contiguous().to(dev)
    layer = encode.compress_kv(k[:, :, :S].to(dev), v[:, :, :S].to(dev), block=64, bits_k=4, bits_v=4, k_rel=1 / 14, v_rel=1 / 14,
                               k_mode=QuantMode.ChannelQuant, repack_method=RepackMethod.MEDIAN, capacity_tokens=2048)
    blob = serialize.dumps_layer(layer)
    assert len(blob) < 0.4 * 2 * B * H * S * 128 * 2          # well under the fp16 size
    back = serialize.loads_layer(blob, dev)
    o1 = ops.decode_attention(q, layer, None, None, 0)
    o2 = ops.decode_attention(q, back, None, None, 0)
    assert torch.equal(o1, o2)

    PackKVCacheConfigStatic.config = PackKVCacheConfig("synthetic", QuantMethod.KIVI, RepackMethod.NONE, False, 64, 192, 16, 1 / 14, 1 / 14)
    try:
        cos, sin = synth.rope_tables(S + 80, 128, device=dev, dtype=dtype)
        kd, vd = k.to(dev), v.to(dev)
        cache = PackKVCache(B, H * G, 128, 1)
        cache.update(kd[:, :, :S], vd[:, :, :S], 0, {"cos": cos[:, :S], "sin": sin[:, :S]})
        twin = serialize.loads_cache(serialize.dumps_cache(cache), dev)
        assert twin.get_seq_length() == cache.get_seq_length() == S
        for t in range(S, S + 80):                               # crosses a block boundary: the restored store grows
            for c in (cache, twin):
                c.update(kd[:, :, t:t + 1], vd[:, :, t:t + 1], 0, {"cos": cos[:, t:t + 1], "sin": sin[:, t:t + 1]})
            assert torch.equal(cache.attend(q.unsqueeze(2), 0), twin.attend(q.unsqueeze(2), 0))
        cache.check_flags(); twin.check_flags()
    finally:
        PackKVCacheConfigStatic.config = None
