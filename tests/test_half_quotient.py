"""The encoder forms x / scale in the element type (HalfQuotient, csrc/quant_dev.cuh).  The claim
that this rounds to the same integer code as the reference's fp32 division is checked exhaustively
by oracle/half_quotient_check.c; the full domain (fp16: scale exponents 5..21, bf16: 100..140)
takes a few minutes on one core, so the default run covers a band of each and the edges, and
PACKKV_FULL_QUOTIENT_CHECK=1 runs everything."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def checker(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("hq") / "half_quotient_check")
    subprocess.run(["gcc", "-O2", "-o", exe, os.path.join(ROOT, "oracle", "half_quotient_check.c"), "-lm"], check=True)
    return exe


FULL = os.environ.get("PACKKV_FULL_QUOTIENT_CHECK") == "1"
CASES = [(0, 5, 21, 128), (1, 100, 140, 1)] if FULL else [(0, 5, 5, 128), (0, 12, 13, 128), (0, 21, 21, 128), (1, 100, 100, 1), (1, 123, 124, 1), (1, 140, 140, 1)]


@pytest.mark.parametrize("bf16,lo,hi,pre", CASES)
def test_integer_codes_match_reference_division(checker, bf16, lo, hi, pre):
    r = subprocess.run([checker, str(bf16), str(lo), str(hi), str(pre)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout
    assert " bad 0 of " in r.stdout and "(scales skipped: 0)" in r.stdout, r.stdout
