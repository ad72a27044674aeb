"""CPU: the codec oracle against the committed golden vectors (made from the reference's own
sources by tests/golden/make_golden.py) and, when it can be built, against the compiled
reference directly."""
import os

import numpy as np
import pytest

from oracle import codec


def _parse(name):
    which, cb, bits, hidden, _ = name.split("_")
    return which, int(cb[2:]), int(bits[1:]), int(hidden[1:])


@pytest.fixture(scope="module")
def golden(golden_dir):
    return np.load(os.path.join(golden_dir, "codec_golden.npz"))


def test_restatement_matches_golden_streams(golden):
    R = codec.restated()
    for name in golden["cases"]:
        which, cb, bits, hidden = _parse(str(name))
        codes = golden[f"{name}_codes"]
        stream, info = R.encode(which, codes, cb, bits)
        assert np.array_equal(stream, golden[f"{name}_stream"]), name
        assert np.array_equal(info, golden[f"{name}_info"]), name
        back = R.decode(which, golden[f"{name}_stream"], golden[f"{name}_info"], codes.shape[0], hidden, cb, bits)
        assert np.array_equal(back, codes), name


def test_restatement_matches_compiled_reference():
    F = codec.reference()
    if F is None:
        pytest.skip("reference checkout / prebuilt oracle/_ref not available")
    R = codec.restated()
    rng = np.random.default_rng(7)
    for which, cbs in (("k", (32, 64, 128)), ("v", (128,))):
        for cb in cbs:
            for bits in (2, 3, 4):
                for hidden in (128, 1024):
                    codes = np.clip(np.round(rng.normal(2 ** bits / 2, 1.2, (2 * cb, hidden))), 0, 2 ** bits - 1).astype(np.uint8)
                    s1, i1 = R.encode(which, codes, cb, bits)
                    s2, i2 = F.encode(which, codes, cb, bits)
                    assert np.array_equal(s1, s2) and np.array_equal(i1, i2)
                    assert np.array_equal(F.decode(which, s1, i1, 2 * cb, hidden, cb, bits), codes)


@pytest.mark.parametrize("which,cb", [("k", 32), ("k", 64), ("k", 128), ("v", 32), ("v", 64), ("v", 128)])
@pytest.mark.parametrize("bits", [2, 3, 4])
def test_round_trip_and_edges(which, cb, bits):
    R = codec.restated()
    rng = np.random.default_rng(cb * 10 + bits)
    hb = 128 if which == "k" else 64
    top = 2 ** bits - 1
    cases = [
        rng.integers(0, top + 1, (3 * cb, 2 * hb), dtype=np.uint8),   # incompressible
        np.zeros((cb, hb), np.uint8),                                 # every len = 0
        np.full((cb, hb), top, np.uint8),                             # constant at the top code
        np.zeros((0, hb), np.uint8),                                  # empty sequence
    ]
    alt = np.zeros((cb, hb), np.uint8)
    alt[::2] = top                                                    # full range in every pack
    cases.append(alt)
    for codes in cases:
        stream, info = R.encode(which, codes, cb, bits)
        nblk = (codes.shape[0] // cb) * (codes.shape[1] // hb)
        assert info.shape == (nblk, 2)
        if nblk:
            assert info[0, 0] == 0 and int(info[-1, 0]) + int(info[-1, 1]) == stream.size
            assert (info[1:, 0] == info[:-1, 0] + info[:-1, 1]).all()        # back to back
            assert int(info[:, 1].max()) <= R.block_bound(which, cb, bits)
        assert np.array_equal(R.decode(which, stream, info, codes.shape[0], codes.shape[1], cb, bits), codes)
    # header-only block when every pack is constant
    s0, i0 = R.encode(which, np.zeros((cb, hb), np.uint8), cb, bits)
    lb = 3 if bits == 4 else 2
    assert s0.size == (2 * (cb // 16) + (cb // 16) * 16 * (bits + lb) if which == "k"
                       else 2 * (4 if cb == 128 else 2) + (cb // 16) * 64 * (bits + lb) // 8)


def test_bad_arguments_are_rejected():
    R = codec.restated()
    with pytest.raises(ValueError):
        R.encode("k", np.zeros((64, 128), np.uint8), 64, 5)
    with pytest.raises(ValueError):
        R.encode("k", np.zeros((48, 128), np.uint8), 64, 4)
    with pytest.raises(ValueError):
        R.encode("v", np.zeros((128, 64), np.uint8), 16, 4)
