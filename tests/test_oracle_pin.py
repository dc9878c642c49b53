"""Pins the CPU oracle (CPU only): the restatement in oracle/halo_oracle.cpp against
(a) the reference's gguf-py golden blocks, (b) its known-answer tests for the half
conversions, (c) the reference's own sources compiled unmodified (bit for bit, when
the checkout is present), and (d) the committed outputs of those sources."""
import numpy as np
import pytest

import oracle
from conftest import GOLDEN
from halo_flash_b200 import synth


def _rows():
    out = []
    for line in (GOLDEN / "quant_blocks.tsv").read_text().splitlines():
        typ, blk, vals = line.split("\t")
        out.append((typ, np.frombuffer(bytes.fromhex(blk), dtype=np.uint8),
                    np.frombuffer(bytes.fromhex(vals), dtype=np.float32)))
    return out


def _decode(o, typ, block, k):
    if typ == "Q8_0":
        return o.embed_q8_0_rows(block.reshape(1, -1), np.zeros(1, np.uint32), k)[0]
    return o.dequant_f16(block) if typ == "F16" else o.dequant_bf16(block)


def test_golden_blocks_count():
    rows = _rows()
    assert len(rows) == 36 and {t for t, _, _ in rows} == {"Q8_0", "F16", "BF16"}


@pytest.mark.parametrize("kind", ["port", "reference"])
def test_decode_matches_gguf_py_blocks(kind):
    """tests/core/quant_test.cpp:253-268 (DequantizeMatchesGgufPy): single blocks and
    two-block rows, within the reference's 4e-7 relative bound; for these formats the
    decode is exact, so equality is asserted as well."""
    if kind == "reference" and not oracle.have_reference():
        pytest.skip("reference library not built here")
    o = oracle.load(kind)
    rows = _rows()
    for i, (typ, block, want) in enumerate(rows):
        got = _decode(o, typ, block, want.size)
        assert np.all(np.abs(got - want) <= 4e-7 * np.abs(want)), (typ, i)
        assert got.tobytes() == want.tobytes(), (typ, i)
        if i + 1 < len(rows) and rows[i + 1][0] == typ:
            two = np.concatenate([block, rows[i + 1][1]])
            want2 = np.concatenate([want, rows[i + 1][2]])
            assert _decode(o, typ, two, want2.size).tobytes() == want2.tobytes(), (typ, i, "two blocks")


def test_fp16_known_answers(port):
    """tests/core/quant_test.cpp:270-281 (Fp16InfinityAndNan) and :103-120 (every finite
    pattern converts to the value its fields denote)."""
    # through the array decoder: a float returned by value would lose a signalling NaN's payload
    bits = lambda h: int(port.dequant_f16(np.array([h], dtype="<u2").view(np.uint8)).view(np.uint32)[0])
    assert bits(0x7C00) == 0x7F800000
    assert bits(0xFC00) == 0xFF800000
    assert bits(0x7E00) == 0x7FC00000
    assert bits(0xFD01) == 0xFFA02000
    assert bits(0x8000) == 0x80000000
    h = np.arange(0x10000, dtype=np.uint32)
    e, m, s = (h >> 10) & 31, h & 1023, h >> 15
    fin = e != 31
    want = np.where(e == 0, np.ldexp(m.astype(np.float64), -24), np.ldexp((1024 + m).astype(np.float64), e.astype(np.int64) - 25))
    want = np.where(s == 1, -want, want)
    got = port.dequant_f16(h.astype("<u2").view(np.uint8)).astype(np.float64)
    assert np.array_equal(got[fin], want[fin])
    # bf16: bits << 16
    b = np.arange(0x10000, dtype=np.uint32)
    gotb = port.dequant_bf16(b.astype("<u2").view(np.uint8)).view(np.uint32)
    assert np.array_equal(gotb, b << 16)


def test_q8_0_is_scale_times_int(port):
    """tests/core/quant_test.cpp:91-101 (Q8_0IsScaleTimesInt)."""
    table = synth.q8_0_table("pin.q8", 64, 256)
    ids = np.arange(64, dtype=np.uint32)
    got = port.embed_q8_0_rows(table, ids, 256)
    blocks = table.reshape(64, 8, 34)
    d = port.dequant_f16(np.ascontiguousarray(blocks[:, :, :2]).reshape(-1)).reshape(64, 8, 1)
    q = blocks[:, :, 2:].view(np.int8).astype(np.float32)
    assert np.array_equal(got.reshape(64, 8, 32), d * q)


def test_q8_0_encode_error_is_half_a_step(port):
    """tests/core/lowbit_test.cpp:138-155 (Q8ContainerErrorIsHalfAStep)."""
    g = synth.rng("pin.enc")
    for cols in (32, 96, 1280):
        x = (0.02 * g.standard_normal((5, cols))).astype(np.float32)
        enc = port.encode_q8_0_rows(x)
        y = np.stack([port.embed_q8_0_rows(enc[r:r + 1], np.zeros(1, np.uint32), cols)[0] for r in range(5)])
        amax = np.abs(x).reshape(5, -1, 32).max(axis=2, keepdims=True)
        err = np.abs(y - x).reshape(5, -1, 32)
        assert np.all(err <= amax / 127.0 * 0.5 * 1.01 + 1e-12)
    zeros = port.encode_q8_0_rows(np.zeros((1, 32), np.float32))
    assert not zeros.any()  # d == 0 -> all codes 0


@pytest.mark.skipif(not oracle.have_reference(), reason="reference library not built here")
def test_port_equals_compiled_reference_bit_for_bit(port):
    ref = oracle.load("reference")
    assert ref.kind == "reference" and port.kind == "port"
    g = synth.rng("pin.eq")
    for d in (8, 64, 100, 256, 2048):
        x = g.standard_normal((9, d)).astype(np.float32) * 3
        w = (1 + 0.1 * g.standard_normal((3, d))).astype(np.float32)
        for eps in (1e-6, 1e-5):
            a = port.rmsnorm_rows(x.copy(), w, eps, w_stride=d, w_period=3)
            b = ref.rmsnorm_rows(x.copy(), w, eps, w_stride=d, w_period=3)
            assert a.tobytes() == b.tobytes()
            assert port.rmsnorm_rows(x.copy(), None, eps).tobytes() == ref.rmsnorm_rows(x.copy(), None, eps).tobytes()
            assert port.l2norm_rows(x.copy(), eps).tobytes() == ref.l2norm_rows(x.copy(), eps).tobytes()
            z = g.standard_normal((9, d)).astype(np.float32) * 4
            for mode in (0, 1):
                assert (port.gated_norm_rows(x.copy(), w[0], z, eps, mode).tobytes()
                        == ref.gated_norm_rows(x.copy(), w[0], z, eps, mode).tobytes())
    for heads, hd, rot, theta in ((4, 64, 16, 1e7), (18, 256, 64, 1e7), (3, 32, 32, 1e4), (2, 24, 6, 5e5)):
        x = g.standard_normal((11, heads, hd)).astype(np.float32)
        pos = g.integers(0, 262144, size=11, dtype=np.uint32)
        pos[0], pos[1] = 0, 262143
        assert port.rope_rows(x.copy(), pos, rot, theta).tobytes() == ref.rope_rows(x.copy(), pos, rot, theta).tobytes()
    a, b = (g.standard_normal(4099).astype(np.float32) * 6 for _ in range(2))
    assert port.silu_mul(a.copy(), b).tobytes() == ref.silu_mul(a.copy(), b).tobytes()
    table = synth.q8_0_table("pin.eq.table", 97, 512)
    ids = g.integers(0, 97, size=40, dtype=np.uint32)
    assert port.embed_q8_0_rows(table, ids, 512).tobytes() == ref.embed_q8_0_rows(table, ids, 512).tobytes()
    x = g.standard_normal((7, 640)).astype(np.float32) * np.float32(10.0) ** g.integers(-6, 4, size=(7, 1))
    x[0, :32] = 0
    assert port.encode_q8_0_rows(x).tobytes() == ref.encode_q8_0_rows(x).tobytes()
    for v in (-30.0, -1.5, 0.0, 0.3, 25.0):
        assert port._call("orc_silu", v) == ref._call("orc_silu", v)


@pytest.mark.parametrize("kind", ["port", "reference"])
def test_committed_reference_outputs(kind, golden_ops):
    """ops_c1.npz was produced by the reference's compiled CPU operators
    (tests/golden/make_golden.py); the checker must reproduce it bit for bit."""
    if kind == "reference" and not oracle.have_reference():
        pytest.skip("reference library not built here")
    o, gd, s = oracle.load(kind), golden_ops, synth.C1
    one = np.float32(1.0)
    summed = gd["res"] + gd["delta"]
    assert summed.tobytes() == gd["res_out"].tobytes()
    xn = o.rmsnorm_rows(summed.copy(), one + gd["norm_w"], s.eps)
    assert xn.tobytes() == gd["xn"].tobytes()
    assert o.encode_q8_0_rows(xn).tobytes() == gd["xn_q8_0"].tobytes()
    assert o.l2norm_rows(gd["qk"].copy(), s.eps).tobytes() == gd["qk_l2"].tobytes()
    assert o.gated_norm_rows(gd["o"].copy(), gd["gated_w"], gd["z"], s.eps, 0).tobytes() == gd["gated_silu"].tobytes()
    assert o.gated_norm_rows(gd["o"].copy(), gd["gated_w"], gd["z"], s.eps, 1).tobytes() == gd["gated_sigmoid"].tobytes()
    assert o.rope_rows(gd["q"].copy(), gd["pos"], s.rot, s.theta).tobytes() == gd["q_rope"].tobytes()
    assert o.rope_rows(gd["k"].copy(), gd["pos"], s.rot, s.theta).tobytes() == gd["k_rope"].tobytes()
    qn = o.rmsnorm_rows(gd["q"].copy(), one + gd["qnorm_w"], s.eps)
    assert o.rope_rows(qn, gd["pos"], s.rot, s.theta).tobytes() == gd["q_norm_rope"].tobytes()
    assert o.silu_mul(gd["gate"].copy(), gd["up"]).tobytes() == gd["swiglu"].tobytes()
    table = np.zeros((s.vocab, s.q8_row_bytes), np.uint8)
    table[gd["table_rows"]] = gd["table_bytes"]
    assert o.embed_q8_0_rows(table, gd["ids"], s.hidden).tobytes() == gd["embed"].tobytes()


def test_synthetic_inputs_are_reproducible(golden_ops):
    """The seeded generators reproduce the committed inputs (same stream on every box)."""
    s = synth.C1
    assert synth.act("g.res", 32, s.hidden).tobytes() == golden_ops["res"].tobytes()
    assert synth.norm_w("g.norm_w", s.hidden).tobytes() == golden_ops["norm_w"].tobytes()
    assert synth.positions("g.pos", 32, s.max_pos).tobytes() == golden_ops["pos"].tobytes()
    assert synth.token_ids("g.ids", 32, s.vocab).tobytes() == golden_ops["ids"].tobytes()
    t = synth.q8_0_table("g.table", s.vocab, s.hidden)
    assert t[golden_ops["table_rows"]].tobytes() == golden_ops["table_bytes"].tobytes()


def test_bf16_helpers_match_port(port):
    x = synth.act("pin.bf16", 4096) * np.float32(1e3)
    want = np.array([port._call("orc_float_to_bf16", float(v)) for v in x[:512]], dtype=np.uint16)
    assert np.array_equal(oracle.bf16_bits(x[:512]), want)
    assert np.array_equal(port.round_bf16(x.copy()), oracle.round_bf16(x))


# ---- the ops around the five groups: hyper-connection residual, experts' combine, DeltaNet conv -------
@pytest.fixture(scope="module")
def golden_wide():
    return np.load(GOLDEN / "ops_wide_c1.npz")


def _wide_outputs(orc, g):
    s = synth.C1
    out = {}
    for name, rnd in (("f32", 0), ("bf16", 1), ("f16", 2)):
        r = g["hc_res"].copy()
        if rnd == 1:
            r = oracle.round_bf16(r)
        if rnd == 2:
            r = r.astype(np.float16).astype(np.float32)
        out[f"hc_y_{name}"] = orc.hc_combine_norm(r, g["hc_out"], g["hc_inject"], g["hc_gamma"], s.eps, rnd)
        out[f"hc_res_out_{name}"] = r
    T = g["hc_res"].shape[0]
    out["hc_inject_proj"] = orc.hc_inject(out["hc_y_f32"].reshape(T, -1), g["hc_iw"])
    out["hc_mixed"] = orc.hc_mix(out["hc_y_f32"], g["hc_gate"])
    out["moe_routed"] = orc.moe_combine(g["moe_yp"], g["moe_pos"], g["moe_w"])
    out["moe_out"] = orc.moe_combine(g["moe_yp"], g["moe_pos"], g["moe_w"], g["moe_sx"], g["moe_sg"])
    st = g["conv_state"].copy()
    l2, d = 2 * s.k_heads * s.lin_dim, s.lin_dim
    out["conv_out"] = orc.conv_l2norm(g["conv_x"], st, g["conv_w"], l2, d, s.eps)
    out["conv_state_out"] = st
    return out


@pytest.mark.parametrize("kind", ["port", "reference"])
def test_committed_reference_outputs_of_the_widened_ops(kind, golden_wide):
    """The port (and, where it is built, the compiled reference) reproduces the committed outputs bit for bit."""
    if kind == "reference" and not oracle.have_reference():
        pytest.skip("reference library not built here")
    got = _wide_outputs(oracle.load(kind), golden_wide)
    for name, value in got.items():
        assert value.tobytes() == golden_wide[name].tobytes(), name


def test_widened_op_identities(port, golden_wide):
    """Relations the CPU operators satisfy by construction (src/model/reference.cpp:189-202, 151-160)."""
    g, s = golden_wide, synth.C1
    T, hc, h = g["hc_res"].shape
    # zero logits: 2 sigmoid(0) = 1, the combine is a plain add into every stream
    r = g["hc_res"].copy()
    port.hc_combine_norm(r, g["hc_out"], np.zeros((T, hc), np.float32), g["hc_gamma"], s.eps, 0)
    assert np.array_equal(r, g["hc_res"] + g["hc_out"][:, None, :])
    # the grouped norm is the plain row norm with gamma row = stream index
    y = port.hc_combine_norm(g["hc_res"].copy(), None, None, g["hc_gamma"], s.eps, 0)
    rows = port.rmsnorm_rows(g["hc_res"].reshape(T * hc, h).copy(), g["hc_gamma"], s.eps, w_stride=h, w_period=hc)
    assert np.array_equal(y.reshape(T * hc, h), rows)
    # the conv of a chunk equals token-by-token stepping with the state carried along
    st_a, st_b = g["conv_state"].copy(), g["conv_state"].copy()
    l2, d = 2 * s.k_heads * s.lin_dim, s.lin_dim
    whole = port.conv_l2norm(g["conv_x"], st_a, g["conv_w"], l2, d, s.eps)
    steps = np.concatenate([port.conv_l2norm(g["conv_x"][t:t + 1], st_b, g["conv_w"], l2, d, s.eps) for t in range(T)])
    assert np.array_equal(whole, steps) and np.array_equal(st_a, st_b)
    assert np.array_equal(st_a, g["conv_x"][-3:])
