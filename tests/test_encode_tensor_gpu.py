"""GPU: the one-call encoder (pkv_encode_tensor: fp16/bf16 -> streams).  For K per-channel and V
per-token it runs the single-pass kernels; everything it writes -- streams, block tables, byte
counts, scales, zero-points -- must equal the CPU oracle (reference quantiser + reference codec)
bit for bit, for every bit width and block size, and must equal the two-stage GPU pipeline."""
import numpy as np
import pytest
import torch

from oracle import codec
from oracle import quant as Q
from packkv_b200 import encode, ops, synth

pytestmark = pytest.mark.gpu


def _bufs(B, H, S, cb, bits, which, mode, dtype, dev, extra_tokens=0):
    cap = S + extra_tokens
    shape = (B, H, cap // cb, 128) if mode == ops.K_CHANNEL else (B, cap)
    return dict(scale=torch.zeros(shape, dtype=dtype, device=dev), zero=torch.zeros(shape, dtype=dtype, device=dev),
                stream=torch.zeros(B, encode.stream_capacity(which, cap, H, cb, bits), dtype=torch.uint8, device=dev),
                info=torch.zeros(B, (cap // cb) * H * (1 if which == "k" else 2), 2, dtype=torch.int32, device=dev),
                stream_bytes=torch.zeros(B, dtype=torch.int32, device=dev), flags=ops.new_flags(dev))


def _oracle(x, which, mode, block, bits, hp):
    c, z, s = Q.quant_ints(x, block, synth.rel_for_bits(bits), "channel" if mode == ops.K_CHANNEL else "token", hp)
    codes = c.flatten(2, 3).permute(0, 2, 1, 3).flatten(2, 3).contiguous().to(torch.uint8)
    R = codec.restated()
    return [R.encode(which, codes[b].numpy(), block, bits) for b in range(x.shape[0])], z, s


@pytest.mark.parametrize("which,mode", [("k", ops.K_CHANNEL), ("v", ops.K_TOKEN), ("k", ops.K_TOKEN)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_encode_tensor_matches_oracle(cuda_device, which, mode, dtype):
    dev = cuda_device
    B, H = 2, 4
    k, v = synth.synth_kv(B, H, 384, 128, seed=41, dtype=dtype, apply_rope=True)
    x = k if which == "k" else v
    for bits in (2, 3, 4):
        for block in (32, 64, 128):
            for hp in (False, True):
                if hp and (bits, block) != (4, 64):
                    continue
                want, z, s = _oracle(x, which, mode, block, bits, hp)
                bufs = _bufs(B, H, 384, block, bits, which, mode, dtype, dev)
                ops.encode_tensor(which, x.to(dev), block, synth.rel_for_bits(bits), mode, bits, block, high_precision_zero=hp, **bufs)
                torch.cuda.synchronize()
                assert int(bufs["flags"].item()) == 0
                for b in range(B):
                    ws, wi = want[b]
                    assert int(bufs["stream_bytes"][b].item()) == ws.size, (bits, block)
                    assert np.array_equal(bufs["stream"][b, : ws.size].cpu().numpy(), ws), (bits, block, hp)
                    assert np.array_equal(bufs["info"][b].cpu().numpy().view(np.uint32), wi)
                shape = bufs["scale"].shape
                assert torch.equal(bufs["scale"].cpu().view(torch.int16), s.reshape(shape).contiguous().view(torch.int16))
                assert torch.equal(bufs["zero"].cpu().view(torch.int16), z.reshape(shape).contiguous().view(torch.int16))


def test_append_in_pieces_equals_one_call_and_flags(cuda_device):
    dev, dtype = cuda_device, torch.float16
    B, H, S = 3, 8, 512
    k, v = synth.synth_kv(B, H, S, 128, seed=43, dtype=dtype, device=dev)
    for which, mode, x in (("k", ops.K_CHANNEL, k), ("v", ops.K_TOKEN, v)):
        one = _bufs(B, H, S, 64, 4, which, mode, dtype, dev)
        ops.encode_tensor(which, x, 64, 1 / 14, mode, 4, 64, **one)
        parts = _bufs(B, H, S, 64, 4, which, mode, dtype, dev)
        for t0, t1 in ((0, 192), (192, 256), (256, 512)):
            ops.encode_tensor(which, x[:, :, t0:t1], 64, 1 / 14, mode, 4, 64, first_token=t0, **parts)
        torch.cuda.synchronize()
        for key in ("scale", "zero", "info", "stream_bytes"):
            assert torch.equal(one[key], parts[key]), key
        for b in range(B):
            n = int(one["stream_bytes"][b].item())
            assert torch.equal(one["stream"][b, :n], parts["stream"][b, :n])
    # codes that do not fit the bit width are reported, a stream that is too small is reported
    bufs = _bufs(B, H, S, 64, 3, "k", ops.K_CHANNEL, dtype, dev)
    ops.encode_tensor("k", k, 64, 0.1, ops.K_CHANNEL, 3, 64, **bufs)
    small = _bufs(B, H, S, 64, 4, "k", ops.K_CHANNEL, dtype, dev)
    small["stream"] = torch.zeros(B, 4096, dtype=torch.uint8, device=dev)
    ops.encode_tensor("k", k, 64, 1 / 14, ops.K_CHANNEL, 4, 64, **small)
    torch.cuda.synchronize()
    assert int(bufs["flags"].item()) & 2 and int(small["flags"].item()) & 1


@pytest.mark.parametrize("layout", ["bshd", "sliced", "padded_heads"])
@pytest.mark.parametrize("which,mode", [("k", ops.K_CHANNEL), ("k", ops.K_TOKEN), ("v", ops.K_TOKEN)])
def test_strided_inputs(cuda_device, layout, which, mode):
    """Inputs that are views of larger or differently ordered buffers (token-major memory, a window of a
    longer sequence, a subset of heads): same bytes as for the contiguous tensor."""
    dev, dtype = cuda_device, torch.bfloat16
    B, H, S, cb, bits = 2, 3, 192, 64, 4
    k, v = synth.synth_kv(B, H, S, 128, seed=47, dtype=dtype, apply_rope=True)
    x = (k if which == "k" else v).to(dev)
    if layout == "bshd":
        xs = x.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    elif layout == "sliced":
        big = torch.zeros(B, H, S + 2 * cb, 128, dtype=dtype, device=dev)
        big[:, :, cb:cb + S] = x
        xs = big[:, :, cb:cb + S]
    else:
        big = torch.zeros(B, H + 2, S, 128, dtype=dtype, device=dev)
        big[:, 1:H + 1] = x
        xs = big[:, 1:H + 1]
    assert not xs.is_contiguous() and torch.equal(xs, x)
    rel = synth.rel_for_bits(bits)
    a, b = _bufs(B, H, S, cb, bits, which, mode, dtype, dev), _bufs(B, H, S, cb, bits, which, mode, dtype, dev)
    ops.encode_tensor(which, x, cb, rel, mode, bits, cb, **a)
    ops.encode_tensor(which, xs, cb, rel, mode, bits, cb, **b)
    torch.cuda.synchronize()
    assert int(a["flags"].item()) == 0 and int(b["flags"].item()) == 0
    for name in ("stream", "info", "stream_bytes", "scale", "zero"):
        assert torch.equal(a[name].view(torch.uint8), b[name].view(torch.uint8)), name


@pytest.mark.parametrize("which,mode", [("k", ops.K_CHANNEL), ("v", ops.K_TOKEN), ("k", ops.K_TOKEN)])
@pytest.mark.parametrize("H,S", [(3, 128), (12, 128), (1, 64), (2, 64 * 150)])
def test_direct_and_slot_forms(cuda_device, which, mode, H, S):
    """The encoder writes blocks straight to the stream after a look-back over the CTAs before it in the sequence;
    with more than 8 heads the per-token kernels go through slots and a compaction pass instead.  Head counts
    that leave the last CTA of a sequence partly empty (3), that take the slot form (12), the smallest input, and
    a sequence long enough for look-backs of more than one 32-entry window (150 token blocks, 75 K CTAs of 4
    blocks): all byte-exact against the oracle, three sequences so that chains of different sequences interleave."""
    dev, dtype = cuda_device, torch.float16
    B, block, bits = 3, 64, 4
    k, v = synth.synth_kv(B, H, S, 128, seed=43, dtype=dtype, apply_rope=True)
    x = k if which == "k" else v
    want, z, s = _oracle(x, which, mode, block, bits, False)
    bufs = _bufs(B, H, S, block, bits, which, mode, dtype, dev)
    for _ in range(2):   # a second call on the same scratch-free interface must start from clean look-back state
        ops.encode_tensor(which, x.to(dev), block, synth.rel_for_bits(bits), mode, bits, block, **bufs)
    torch.cuda.synchronize()
    assert int(bufs["flags"].item()) == 0
    for b in range(B):
        ws, wi = want[b]
        assert int(bufs["stream_bytes"][b].item()) == ws.size
        assert np.array_equal(bufs["stream"][b, : ws.size].cpu().numpy(), ws)
        assert np.array_equal(bufs["info"][b].cpu().numpy().view(np.uint32), wi)
