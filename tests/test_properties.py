"""Property tests on CPU (hypothesis), in the spirit of the reference's property tests of its quantizers
(tests/core/quant_test.cpp): the port of each CPU operator equals the compiled reference on arbitrary small
shapes, and the relations the operators satisfy by construction hold for arbitrary inputs."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

import oracle
from halo_flash_b200 import chain

PORT = oracle.load("port")
REF = oracle.load("reference") if oracle.have_reference() else None
SETTINGS = dict(max_examples=40, deadline=None, derandomize=True)  # the same examples on every run


def arr(rng, *shape, scale=3.0):
    return (rng.standard_normal(shape) * scale).astype(np.float32)


@given(total=st.integers(0, 1 << 20), world=st.integers(1, 16))
@settings(**SETTINGS)
def test_shards_partition_the_tokens(total, world):
    spans = [chain.shard_range(total, r, world) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == total
    assert all(e0 == b1 for (_, e0), (b1, _) in zip(spans, spans[1:]))
    sizes = [e - b for b, e in spans]
    assert max(sizes) - min(sizes) <= 1 and sorted(sizes, reverse=True) == sizes


@given(seed=st.integers(0, 2**32 - 1), tokens=st.integers(1, 5), hc=st.integers(1, 5), h=st.integers(1, 70),
       rnd=st.sampled_from([0, 1, 2]))
@settings(**SETTINGS)
def test_hc_ops_port_equals_reference(seed, tokens, hc, h, rnd):
    if REF is None:
        pytest.skip("reference library not built here")
    rng = np.random.default_rng(seed)
    res, out, inj = arr(rng, tokens, hc, h), arr(rng, tokens, h), arr(rng, tokens, hc)
    w = (1 + 0.1 * rng.standard_normal((hc, h))).astype(np.float32)
    ra, rb = res.copy(), res.copy()
    ya, yb = PORT.hc_combine_norm(ra, out, inj, w, 1e-6, rnd), REF.hc_combine_norm(rb, out, inj, w, 1e-6, rnd)
    assert ra.tobytes() == rb.tobytes() and ya.tobytes() == yb.tobytes()
    gate = arr(rng, tokens, hc, h)
    assert PORT.hc_mix(ya, gate).tobytes() == REF.hc_mix(ya, gate).tobytes()
    iw = arr(rng, 3, hc * h, scale=0.1)
    assert PORT.hc_inject(ya.reshape(tokens, -1), iw).tobytes() == REF.hc_inject(ya.reshape(tokens, -1), iw).tobytes()


@given(seed=st.integers(0, 2**32 - 1), tokens=st.integers(1, 9), heads=st.integers(1, 4), d=st.integers(1, 24),
       l2_heads=st.integers(0, 4), kern=st.integers(1, 6))
@settings(**SETTINGS)
def test_conv_port_equals_reference_and_steps(seed, tokens, heads, d, l2_heads, kern):
    rng = np.random.default_rng(seed)
    C, l2 = heads * d, min(l2_heads, heads) * d
    x, st0, w = arr(rng, tokens, C), arr(rng, max(kern - 1, 1), C)[:kern - 1].copy(), arr(rng, C, kern, scale=0.5)
    sa = st0.copy()
    whole = PORT.conv_l2norm(x, sa, w, l2, d, 1e-6)
    if REF is not None:
        sb = st0.copy()
        assert REF.conv_l2norm(x, sb, w, l2, d, 1e-6).tobytes() == whole.tobytes() and sa.tobytes() == sb.tobytes()
    sc = st0.copy()
    steps = np.concatenate([PORT.conv_l2norm(x[t:t + 1], sc, w, l2, d, 1e-6) for t in range(tokens)])
    assert steps.tobytes() == whole.tobytes() and sc.tobytes() == sa.tobytes()
    if l2:
        n = (whole[:, :l2].reshape(tokens, -1, d).astype(np.float64) ** 2).sum(axis=2)
        assert np.all(n <= 1 + 1e-4)  # x / sqrt(sum x^2 + eps): at most unit length, exactly so only as eps -> 0


@given(seed=st.integers(0, 2**32 - 1), tokens=st.integers(1, 6), k=st.integers(1, 12), n=st.integers(1, 40))
@settings(**SETTINGS)
def test_moe_combine_is_linear_in_the_weights(seed, tokens, k, n):
    rng = np.random.default_rng(seed)
    yp, pos = arr(rng, tokens * k, n), rng.permutation(tokens * k).reshape(tokens, k).astype(np.uint32)
    mw = rng.random((tokens, k), dtype=np.float32)
    a = PORT.moe_combine(yp, pos, mw)
    if REF is not None:
        assert REF.moe_combine(yp, pos, mw).tobytes() == a.tobytes()
    assert PORT.moe_combine(yp, pos, (mw * np.float32(2)).astype(np.float32)).tobytes() == (a * np.float32(2)).tobytes()
    one_hot = np.zeros((tokens, k), np.float32)
    one_hot[:, 0] = 1
    assert np.array_equal(PORT.moe_combine(yp, pos, one_hot), yp[pos[:, 0]])
