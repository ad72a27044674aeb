"""GPU: the single-pass encoder on value distributions chosen to reach every quantiser path --
the element-type quotient (ordinary data), the fp32 two-element path (scales or magnitudes outside
the element-type domain), the scalar exact-division path (large zero-points), zeros and fp16
subnormals -- always bit-exact against the reference quantiser + codec on the CPU."""
import numpy as np
import pytest
import torch

from oracle import codec
from oracle import quant as Q
from packkv_b200 import _lib, encode, ops, synth

pytestmark = pytest.mark.gpu


def _make(name, dtype, g):
    shape = (2, 2, 128, 128)
    n = torch.randn(shape, generator=g)
    if name == "normal":
        x = n
    elif name == "tiny":
        x = n * 1e-3
    elif name == "huge":
        x = n * 200.0
    elif name == "offset":
        x = n + 30.0
    elif name == "far_offset":
        x = n * 0.05 + 20.0
    elif name == "sparse":
        x = n * (torch.rand(shape, generator=g) > 0.9)
    elif name == "subnormal":
        x = n * 2e-5
    elif name == "heavy_tail":
        x = (n / (torch.randn(shape, generator=g).abs() + 0.05)).clamp(-3000, 3000)
    elif name == "mixed_channels":
        x = n * torch.exp(2.0 * torch.randn(1, 2, 1, 128, generator=g))
    else:
        raise KeyError(name)
    return x.to(dtype)


NAMES = ["normal", "tiny", "huge", "offset", "far_offset", "sparse", "subnormal", "heavy_tail", "mixed_channels"]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("name", NAMES)
def test_streams_and_parameters_bit_exact(cuda_device, name, dtype):
    g = torch.Generator().manual_seed(NAMES.index(name) + 100)
    x = _make(name, dtype, g)
    B, H, S, _ = x.shape
    R = codec.restated()
    checked = 0
    for which, mode, mname in (("k", ops.K_CHANNEL, "channel"), ("k", ops.K_TOKEN, "token"), ("v", ops.K_TOKEN, "token")):
        for bits in (4, 2):
            rel = synth.rel_for_bits(bits)
            c, z, s = Q.quant_ints(x, 64, rel, mname)
            if not bool(torch.isfinite(c.float()).all()) or float(c.float().min()) < 0 or float(c.float().max()) > 2 ** bits - 1:
                continue        # the reference itself leaves the code range here (constant group or rounding at the edge): flagged, not compared
            codes = c.flatten(2, 3).permute(0, 2, 1, 3).flatten(2, 3).contiguous().to(torch.uint8)
            shape = (B, H, S // 64, 128) if mode == ops.K_CHANNEL else (B, S)
            bufs = dict(scale=torch.zeros(shape, dtype=dtype, device=cuda_device), zero=torch.zeros(shape, dtype=dtype, device=cuda_device),
                        stream=torch.zeros(B, encode.stream_capacity(which, S, H, 64, bits), dtype=torch.uint8, device=cuda_device),
                        info=torch.zeros(B, (S // 64) * H * (1 if which == "k" else 2), 2, dtype=torch.int32, device=cuda_device),
                        stream_bytes=torch.zeros(B, dtype=torch.int32, device=cuda_device), flags=ops.new_flags(cuda_device))
            ops.encode_tensor(which, x.to(cuda_device), 64, rel, mode, bits, 64, **bufs)
            torch.cuda.synchronize()
            assert int(bufs["flags"].item()) == 0, (which, mname, bits)
            assert torch.equal(bufs["scale"].cpu().view(torch.int16), s.reshape(shape).contiguous().view(torch.int16)), (which, mname, bits)
            assert torch.equal(bufs["zero"].cpu().view(torch.int16), z.reshape(shape).contiguous().view(torch.int16)), (which, mname, bits)
            for b in range(B):
                ws, wi = R.encode(which, codes[b].numpy(), 64, bits)
                assert int(bufs["stream_bytes"][b].item()) == ws.size, (which, mname, bits)
                assert np.array_equal(bufs["stream"][b, : ws.size].cpu().numpy(), ws), (which, mname, bits)
            checked += 1
    assert checked >= 2, "the distribution must keep the reference inside the code range for most modes"
