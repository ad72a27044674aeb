"""GPU: the bit-pack encoder/decoder kernels, called through the C ABI, against the CPU
oracle -- byte-exact streams and block_info, golden fixtures, edge cases, append."""
import os

import numpy as np
import pytest
import torch

from oracle import codec
from packkv_b200 import ops

pytestmark = pytest.mark.gpu


def _codes(rng, kind, ctx, hidden, bits):
    top = 2 ** bits
    if kind == "uniform":
        return rng.integers(0, top, (ctx, hidden), dtype=np.uint8)
    if kind == "normal":
        return np.clip(np.round(rng.normal(top / 2, 1.0, (ctx, hidden))), 0, top - 1).astype(np.uint8)
    if kind == "narrow":
        return np.clip(np.round(rng.normal(top / 2, 0.4, (ctx, hidden))), 0, top - 1).astype(np.uint8)
    if kind == "const":
        return np.full((ctx, hidden), top - 1, dtype=np.uint8)
    raise ValueError(kind)


def _gpu_encode(which, codes_np, cb, bits, dev):
    codes = torch.from_numpy(codes_np).to(dev)
    if codes.dim() == 2:
        codes = codes.unsqueeze(0)
    stream, info, nbytes, flags = ops.encode_codes(which, codes.contiguous(), cb, bits)
    torch.cuda.synchronize()
    return stream, info, nbytes, flags


@pytest.mark.parametrize("which,cb", [("k", 32), ("k", 64), ("k", 128), ("v", 32), ("v", 64), ("v", 128)])
@pytest.mark.parametrize("bits", [2, 3, 4])
def test_encode_decode_matches_oracle(which, cb, bits, cuda_device):
    R = codec.restated()
    rng = np.random.default_rng(100 * cb + bits)
    hb = ops.HB[which]
    for kind in ("uniform", "normal", "narrow", "const"):
        for hidden in (hb, 1024):
            ctx = 3 * cb
            codes = _codes(rng, kind, ctx, hidden, bits)
            ref_stream, ref_info = R.encode(which, codes, cb, bits)
            stream, info, nbytes, flags = _gpu_encode(which, codes, cb, bits, cuda_device)
            assert int(flags.item()) == 0
            assert int(nbytes[0].item()) == ref_stream.size
            assert np.array_equal(info[0].cpu().numpy().view(np.uint32), ref_info)
            assert np.array_equal(stream[0, : ref_stream.size].cpu().numpy(), ref_stream), (kind, hidden)
            back, dflags = ops.decode_codes(which, stream, info, ctx, hidden, cb, bits, valid_bytes=ref_stream.size)
            torch.cuda.synchronize()
            assert int(dflags.item()) == 0
            assert np.array_equal(back[0].cpu().numpy(), codes)


def test_golden_streams(cuda_device, golden_dir):
    g = np.load(os.path.join(golden_dir, "codec_golden.npz"))
    for name in g["cases"]:
        which, cb, bits, hidden, _ = str(name).split("_")
        cb, bits, hidden = int(cb[2:]), int(bits[1:]), int(hidden[1:])
        codes = g[f"{name}_codes"]
        stream, info, nbytes, flags = _gpu_encode(which, codes, cb, bits, cuda_device)
        want = g[f"{name}_stream"]
        assert int(nbytes[0].item()) == want.size, name
        assert np.array_equal(stream[0, : want.size].cpu().numpy(), want), name
        assert np.array_equal(info[0].cpu().numpy().view(np.uint32), g[f"{name}_info"]), name
        # decode the reference's bytes
        s = torch.from_numpy(np.concatenate([want, np.zeros(16, np.uint8)])).to(cuda_device).unsqueeze(0)
        i = torch.from_numpy(g[f"{name}_info"].view(np.int32)).to(cuda_device).unsqueeze(0)
        back, dflags = ops.decode_codes(which, s, i, codes.shape[0], hidden, cb, bits, valid_bytes=want.size)
        torch.cuda.synchronize()
        assert int(dflags.item()) == 0 and np.array_equal(back[0].cpu().numpy(), codes), name


def test_batched_sequences_and_append(cuda_device):
    R = codec.restated()
    rng = np.random.default_rng(5)
    for which, cb in (("k", 64), ("v", 128), ("v", 64)):
        n_seq, hidden, bits = 3, 256, 4
        full = np.stack([_codes(rng, "normal", 4 * cb, hidden, bits) for _ in range(n_seq)])
        # prefill with the first 3 blocks, then append the 4th
        head = torch.from_numpy(full[:, : 3 * cb]).to(cuda_device).contiguous()
        tail = torch.from_numpy(full[:, 3 * cb:]).to(cuda_device).contiguous()
        nhid = hidden // ops.HB[which]
        info = torch.zeros(n_seq, 4 * nhid, 2, dtype=torch.int32, device=cuda_device)
        stream = torch.zeros(n_seq, 4 * nhid * ops.block_bound(which, cb, bits), dtype=torch.uint8, device=cuda_device)
        _, _, nbytes, flags = ops.encode_codes(which, head, cb, bits, stream=stream, info=info)
        ops.encode_codes(which, tail, cb, bits, stream=stream, info=info, stream_bytes=nbytes, flags=flags, first_cb=3)
        torch.cuda.synchronize()
        assert int(flags.item()) == 0
        for s in range(n_seq):
            ref_stream, ref_info = R.encode(which, full[s], cb, bits)
            assert int(nbytes[s].item()) == ref_stream.size
            assert np.array_equal(info[s].cpu().numpy().view(np.uint32), ref_info)
            assert np.array_equal(stream[s, : ref_stream.size].cpu().numpy(), ref_stream)


def test_empty_overflow_and_bad_arguments(cuda_device):
    # empty sequence: nothing launched, nothing written
    codes = torch.zeros(1, 0, 128, dtype=torch.uint8, device=cuda_device)
    stream, info, nbytes, flags = ops.encode_codes("k", codes, 64, 4)
    torch.cuda.synchronize()
    assert info.shape[1] == 0 and int(nbytes.item()) == 0 and int(flags.item()) == 0
    # stream too small: blocks that do not fit are skipped and flagged, no out-of-bounds write
    codes = torch.randint(0, 16, (1, 128, 128), dtype=torch.uint8, device=cuda_device)
    small = torch.zeros(1, 5000, dtype=torch.uint8, device=cuda_device)
    guard = small.clone()
    _, _, nbytes, flags = ops.encode_codes("k", codes, 64, 4, stream=small)
    torch.cuda.synchronize()
    assert int(flags.item()) & 1
    # code out of range for the bit width is reported
    bad = torch.full((1, 64, 128), 9, dtype=torch.uint8, device=cuda_device)
    _, _, _, flags = ops.encode_codes("k", bad, 64, 3)
    torch.cuda.synchronize()
    assert int(flags.item()) & 2
    # unsupported geometry -> the reference's "not supported"
    with pytest.raises(RuntimeError, match="not supported"):
        ops.encode_codes("k", torch.zeros(1, 64, 128, dtype=torch.uint8, device=cuda_device), 64, 5)
    with pytest.raises(ValueError):
        ops.encode_codes("k", torch.zeros(1, 48, 128, dtype=torch.uint8, device=cuda_device), 64, 4)
    # corrupt block_info is flagged by the decoder instead of read out of bounds
    codes = torch.randint(0, 16, (1, 64, 128), dtype=torch.uint8, device=cuda_device)
    stream, info, nbytes, flags = ops.encode_codes("k", codes, 64, 4)
    info2 = info.clone()
    info2[0, 0, 0] = 1 << 30
    _, dflags = ops.decode_codes("k", stream, info2, 64, 128, 64, 4)
    torch.cuda.synchronize()
    assert int(dflags.item()) & 4


def test_large_round_trip_property(cuda_device):
    """Full-size property check (no oracle): decode(encode(x)) == x, offsets back to back."""
    torch.manual_seed(0)
    for which, cb, bits in (("k", 64, 4), ("v", 128, 4), ("k", 128, 2)):
        codes = torch.randint(0, 2 ** bits, (4, 8192, 1024), dtype=torch.uint8, device=cuda_device)
        codes = torch.minimum(codes, torch.randint(0, 2 ** bits, (4, 8192, 1), dtype=torch.uint8, device=cuda_device))
        stream, info, nbytes, flags = ops.encode_codes(which, codes, cb, bits)
        back, dflags = ops.decode_codes(which, stream, info, 8192, 1024, cb, bits)
        torch.cuda.synchronize()
        assert int(flags.item()) == 0 and int(dflags.item()) == 0
        assert torch.equal(back, codes)
        i = info.cpu().numpy().view(np.uint32).astype(np.int64)
        assert (i[:, 1:, 0] == i[:, :-1, 0] + i[:, :-1, 1]).all()
        assert (i[:, -1, 0] + i[:, -1, 1] == nbytes.cpu().numpy()).all()
