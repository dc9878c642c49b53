"""pytest configuration: the `gpu` marker, shared fixtures and tolerance helpers.

`-m "not gpu"` covers the oracle against its golden vectors, the host logic and the
C-ABI surface; `-m gpu` holds the parity tests, which call the CUDA kernels through
the C ABI and compare with the oracle on the same seeded inputs.
"""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    # GPU tests are skipped, not failed, where no device is visible (the CPU container).
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def port():
    import oracle
    oracle.build(ref=False) if not oracle.PORT_LIB.exists() else None
    return oracle.load("port")


@pytest.fixture(scope="session")
def orc():
    """The checker: the reference's own compiled CPU operators when present, else the port."""
    import oracle
    if not oracle.PORT_LIB.exists():
        oracle.build(ref=False)
    return oracle.best()


@pytest.fixture(scope="session")
def golden_ops():
    return dict(np.load(GOLDEN / "ops_c1.npz"))


# ---- tolerances (stated once, used by every parity test) ---------------------
def assert_rows_close(got, want, rel=1e-5, what=""):
    """fp32 contract: per-row relative L2 <= rel and |diff| <= rel * max(|want|, rms(want row))."""
    got = np.asarray(got, dtype=np.float64).reshape(-1, got.shape[-1])
    want = np.asarray(want, dtype=np.float64).reshape(-1, want.shape[-1])
    assert got.shape == want.shape, what
    diff = np.abs(got - want)
    rms = np.sqrt(np.mean(want * want, axis=1, keepdims=True))
    bound = rel * np.maximum(np.abs(want), rms) + 1e-30
    bad = diff > bound
    assert not bad.any(), f"{what}: {bad.sum()} elements outside {rel} (max diff {diff.max():.3e})"
    num = np.sqrt((diff * diff).sum(axis=1))
    den = np.sqrt((want * want).sum(axis=1)) + 1e-30
    assert (num / den).max() <= rel, f"{what}: row rel-L2 {(num / den).max():.3e} > {rel}"


def bf16_ordinal(bits):
    """Map bf16 bit patterns to integers ordered like the values (for ulp distances)."""
    b = np.asarray(bits, dtype=np.uint16).astype(np.int32)
    return np.where(b & 0x8000, 0x8000 - (b & 0x7FFF) - 1, 0x8000 + b)


def assert_bf16_within_1ulp(got_bits, want_f32, what=""):
    """bf16 contract: the kernel's bf16 is within 1 bf16 ulp of bf16_rne(oracle fp32)."""
    import oracle
    want_bits = oracle.bf16_bits(np.asarray(want_f32, dtype=np.float32))
    d = np.abs(bf16_ordinal(np.asarray(got_bits).reshape(-1)) - bf16_ordinal(want_bits.reshape(-1)))
    assert d.max() <= 1, f"{what}: {int((d > 1).sum())} values more than 1 bf16 ulp off (max {int(d.max())})"


def assert_bf16_rope(got_bits, want_f32, what=""):
    """bf16 contract for rotated values. A rotated value a*c - b*s can cancel to far below |a|, |b|,
    where the fp32 contract (|diff| <= 1e-5 * max(|a|, |b|)) is many bf16 ulps of the small result.
    So: within 1 bf16 ulp of bf16_rne(oracle), or within 1e-5 of the row's largest magnitude plus
    the bf16 rounding of the value itself."""
    import oracle
    want = np.asarray(want_f32, dtype=np.float32)
    got = oracle.bf16_to_f32(np.asarray(got_bits).reshape(want.shape))
    want_bits = oracle.bf16_bits(want)
    ulps = np.abs(bf16_ordinal(np.asarray(got_bits).reshape(-1)) - bf16_ordinal(want_bits.reshape(-1))).reshape(want.shape)
    rowmax = np.abs(want).max(axis=-1, keepdims=True)
    slack = 1e-5 * rowmax + np.abs(want) * 2.0 ** -8
    bad = (ulps > 1) & (np.abs(got.astype(np.float64) - want) > slack)
    assert not bad.any(), f"{what}: {int(bad.sum())} rotated values outside both bounds"
