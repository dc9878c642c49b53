"""Host-side proofs of arithmetic shortcuts the CUDA kernels take where the contract is bit-exactness.

The Q8 encoders need amax / 127.0f exactly as the CPU computes it (src/core/lowbit.cpp:291). The device code
replaces the division by a multiply and two fused multiply-adds (csrc/common.cuh: div127). tests/cpu/div127_check.c
evaluates that recipe with the C library's correctly rounded fmaf and compares it with the IEEE division.
The whole positive range was checked once (2^31 - 2^23 patterns, zero mismatches); the suite repeats the parts that
decide it: every subnormal and the smallest normals (where the quotient is subnormal), one whole binade of
significands, every 97th pattern of all the others, and the largest finite values.
"""
import shutil
import subprocess
from pathlib import Path

import pytest

SRC = Path(__file__).resolve().parent / "cpu" / "div127_check.c"


@pytest.fixture(scope="module")
def checker(tmp_path_factory):
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    exe = tmp_path_factory.mktemp("div127") / "div127_check"
    subprocess.run([cc, "-O2", "-ffp-contract=off", "-o", str(exe), str(SRC), "-lm"], check=True)
    return exe


@pytest.mark.parametrize("lo,hi,stride", [
    (0x00000000, 0x05000000, 1),      # zero, every subnormal, the normals whose quotient is subnormal or barely normal
    (0x3F800000, 0x40000000, 1),      # every significand of one binade
    (0x05000000, 0x7F000000, 97),     # the rest of the finite range, every 97th pattern
    (0x7F000000, 0x7F800000, 1),      # the top binade up to FLT_MAX
])
def test_fma_quotient_equals_division_by_127(checker, lo, hi, stride):
    out = subprocess.run([str(checker), f"{lo:x}", f"{hi:x}", str(stride)], check=True, capture_output=True, text=True).stdout
    n, bad, first = out.split()
    assert int(n) > 0 and int(bad) == 0, f"{bad} mismatches, first at bit pattern 0x{first}"
