"""GPU: the allocation-free encoder entry point (pkv_encode_tensor_static).

It exists for callers that cannot go to the device allocator in the middle of a decode step -- an
inference server whose block pool took all free HBM at start-up, where a late allocation may fail
and always stalls the device.  Instead of caller scratch it stages the codes in an array built
into the library.  The test drives it through the C ABI twice in a row on different data (the
array keeps the previous call's bytes, which must not leak into the next result) and requires
streams, block tables, byte counts, scales and zero-points identical to the ordinary entry point,
then checks that an over-sized call is refused rather than overrunning the array.

Collected last on purpose: a failure here cannot hide the rest of the suite under `-x`.
"""
import pytest
import torch

from packkv_b200 import _lib, encode, ops, synth

pytestmark = pytest.mark.gpu


def _buffers(B, H, S, block, bits, which, mode, dtype, dev):
    cb = block
    scale_shape = (B, H, S // block, 128) if mode == ops.K_CHANNEL else (B, S)
    return dict(
        scale=torch.zeros(scale_shape, dtype=dtype, device=dev), zero=torch.zeros(scale_shape, dtype=dtype, device=dev),
        stream=torch.zeros(B, encode.stream_capacity(which, S, H, cb, bits), dtype=torch.uint8, device=dev),
        info=torch.zeros(B, (S // cb) * H * (1 if which == "k" else 2), 2, dtype=torch.int32, device=dev),
        stream_bytes=torch.zeros(B, dtype=torch.int32, device=dev), flags=ops.new_flags(dev))


def _same(a, b):
    for key in ("scale", "zero", "info", "stream_bytes", "flags"):
        assert torch.equal(a[key], b[key]), key
    for s in range(a["stream"].shape[0]):
        n = int(a["stream_bytes"][s].item())
        assert torch.equal(a["stream"][s, :n], b["stream"][s, :n])


def test_static_scratch_matches_caller_scratch_twice(cuda_device):
    dev = cuda_device
    calls = [  # (which, mode, dtype, B, H, S, block, bits, seed)
        ("k", ops.K_CHANNEL, torch.bfloat16, 4, 8, 256, 64, 4, 1),
        ("v", ops.K_TOKEN, torch.float16, 2, 4, 128, 64, 3, 2),     # smaller: stale bytes of call 1 stay behind it
    ]
    for which, mode, dtype, B, H, S, block, bits, seed in calls:
        k, v = synth.synth_kv(B, H, S, 128, seed=seed, dtype=dtype, device=dev)
        x = k if which == "k" else v
        rel = synth.rel_for_bits(bits)
        want = _buffers(B, H, S, block, bits, which, mode, dtype, dev)
        got = _buffers(B, H, S, block, bits, which, mode, dtype, dev)
        ops.encode_tensor(which, x, block, rel, mode, bits, block, **want)
        ops.encode_tensor_static(which, x, block, rel, mode, bits, block, **got)
        torch.cuda.synchronize()
        assert int(want["flags"].item()) == 0
        assert int(want["stream_bytes"].min().item()) > 0
        _same(want, got)


def test_static_scratch_two_stage_paths_appends_and_the_exact_limit(cuda_device):
    """The paths that keep a whole code matrix in the built-in array (high-precision zero-points; per-token K),
    an append into a stream that already holds blocks (first_token > 0), and a call that needs exactly the
    array's 16 MiB: all bit-identical to the ordinary entry point."""
    dev = cuda_device
    cases = [  # (which, mode, dtype, B, H, S, block, bits, hp, first_tokens)
        ("k", ops.K_CHANNEL, torch.float16, 2, 4, 256, 64, 4, True, 0),
        ("v", ops.K_TOKEN, torch.bfloat16, 2, 4, 256, 64, 4, True, 0),
        ("k", ops.K_TOKEN, torch.bfloat16, 3, 2, 128, 64, 3, False, 0),
        ("k", ops.K_CHANNEL, torch.bfloat16, 2, 8, 128, 64, 4, False, 128),    # second call appends 128 tokens after 128
        ("k", ops.K_CHANNEL, torch.float16, 4, 8, 4096, 64, 4, False, 0),       # 4*4096*8*128 = 16 MiB exactly
    ]
    for which, mode, dtype, B, H, S, block, bits, hp, first in cases:
        total = S + first
        k, v = synth.synth_kv(B, H, total, 128, seed=11, dtype=dtype, device=dev)
        x = k if which == "k" else v
        rel = synth.rel_for_bits(bits)
        want = _buffers(B, H, total, block, bits, which, mode, dtype, dev)
        got = _buffers(B, H, total, block, bits, which, mode, dtype, dev)
        if S * B * H * 128 == _lib.STATIC_SCRATCH_BYTES:
            assert B * S * H * 128 == _lib.STATIC_SCRATCH_BYTES
        for fn, bufs in ((ops.encode_tensor, want), (ops.encode_tensor_static, got)):
            if first:
                fn(which, x[:, :, :first], block, rel, mode, bits, block, high_precision_zero=hp, **bufs)
            fn(which, x[:, :, first:], block, rel, mode, bits, block, high_precision_zero=hp, first_token=first, **bufs)
        torch.cuda.synchronize()
        assert int(want["flags"].item()) == 0
        assert int(want["stream_bytes"].min().item()) > 0
        _same(want, got)


def test_static_scratch_refuses_oversized_calls(cuda_device):
    dev = cuda_device
    B, H, S = 8, 8, 4096                      # 8*4096*8*128 = 32 MiB of codes > 16 MiB
    assert B * S * H * 128 > _lib.STATIC_SCRATCH_BYTES
    x = torch.zeros(B, H, S, 128, dtype=torch.float16, device=dev)
    bufs = _buffers(B, H, S, 64, 4, "k", ops.K_CHANNEL, torch.float16, dev)
    before = bufs["stream_bytes"].clone()
    with pytest.raises(ValueError, match="built-in scratch"):
        ops.encode_tensor_static("k", x, 64, 1 / 14, ops.K_CHANNEL, 4, 64, **bufs)
    torch.cuda.synchronize()
    assert torch.equal(bufs["stream_bytes"], before)          # nothing was launched
