"""Edges of the parity suite (GPU only): the benchmark's own full-size seeded inputs checked on every row,
the whole argument range of the gate functions, shard invariance of the CUDA op chain, and negative
controls showing that the tolerances in use reject the reference's own planted mutants of this path
(tests/mutants.toml: k-scale-silu-scale, k-rope-sign, k-l2norm-as-rms).
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_bf16_rope, assert_bf16_within_1ulp, assert_rows_close
from halo_flash_b200 import chain as chain_mod, lib, ops, synth

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ONE = np.float32(1.0)
THREADS = 8


def to_dev(a, dtype=None):
    if dtype == "bf16":
        return torch.from_numpy(oracle.bf16_bits(a).view(np.int16)).to(DEV).view(torch.bfloat16).reshape(a.shape)
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def f32(t):
    return t.detach().float().cpu().numpy()


def bits16(t):
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


# ---- the contract's full-size inputs, every row ---------------------------------------------------
def test_full_size_seeded_inputs_every_row(orc):
    """T = 4096 rows of hidden 2048 drawn from the numpy PCG64 stream of the benchmark contract
    (seed 20261125; the tensors the oracle and the CPU arm see), bf16. Residual sum bit-exact on every
    row, xn within 1e-5 on every row, and the Q8_0 epilogue two-stage on every row: scale bits and all
    32 codes of each of the 262 144 blocks equal the CPU encoder applied to the GPU's own fp32 xn."""
    s, T = synth.FULL, 4096
    res = oracle.round_bf16(synth.act("c3.res", T, s.hidden))
    delta = oracle.round_bf16(synth.act("c3.delta", T, s.hidden))
    w = synth.norm_w("c3.w", s.hidden)
    dres, ddelta, dw = to_dev(res, "bf16"), to_dev(delta, "bf16"), to_dev(w)
    xn = torch.empty(T, s.hidden, device=DEV)
    q8 = torch.empty(T, s.q8_row_bytes, dtype=torch.uint8, device=DEV)
    ops.add_rmsnorm(dres, ddelta, dw, s.eps, xn=xn, q8_0=q8)
    stored = oracle.round_bf16(res + delta)
    assert np.array_equal(bits16(dres), oracle.bf16_bits(stored)), "stored residual"
    own = f32(xn)
    assert_rows_close(own, orc.rmsnorm_rows(stored.copy(), ONE + w, s.eps, threads=THREADS), what="full-size xn")
    assert q8.cpu().numpy().tobytes() == orc.encode_q8_0_rows(own, threads=THREADS).tobytes(), "full-size Q8_0 blocks"
    # the decode configuration's form (Q8_0 as the only normalized output) and the bf16 xn form of the same rows
    q8_only = torch.empty_like(q8)
    ops.add_rmsnorm(to_dev(res, "bf16"), ddelta, dw, s.eps, q8_0=q8_only)
    assert torch.equal(q8_only, q8), "Q8_0-only launch differs from the launch that also writes xn"
    xn16 = torch.empty(T, s.hidden, device=DEV, dtype=torch.bfloat16)
    ops.add_rmsnorm(to_dev(res, "bf16"), ddelta, dw, s.eps, xn=xn16)
    assert np.array_equal(bits16(xn16), oracle.bf16_bits(own)), "bf16 xn is the rounding of the fp32 xn"


def test_full_size_seeded_deltanet_and_rope_rows(orc):
    """Configs 3 / 4 on the contract's stream: gated norm (32 x 128), q/k L2 norm (2 x 16 x 128), fused Q/K
    norm + RoPE (16 + 2 heads x 256), SwiGLU rows, bf16 in and out, every row against the oracle."""
    s, T = synth.FULL, 4096
    o = oracle.round_bf16(synth.act("c4.o", T * s.v_heads, s.lin_dim))
    z = oracle.round_bf16(synth.act("c4.z", T * s.v_heads, s.lin_dim))
    gw = synth.gated_w("c4.gw", s.lin_dim)
    y = torch.empty(T * s.v_heads, s.lin_dim, device=DEV, dtype=torch.bfloat16)
    ops.gated_norm(to_dev(o, "bf16"), to_dev(gw), to_dev(z, "bf16"), s.eps, y=y)
    assert_bf16_within_1ulp(bits16(y), orc.gated_norm_rows(o.copy(), gw, z, s.eps, 0, threads=THREADS), "gated norm")
    qk = oracle.round_bf16(synth.act("c4.qk", T * 2 * s.k_heads, s.lin_dim))
    dqk = to_dev(qk, "bf16")
    ops.l2norm(dqk, s.eps)
    assert_bf16_within_1ulp(bits16(dqk), orc.l2norm_rows(qk.copy(), s.eps, threads=THREADS), "q/k L2 norm")
    g = oracle.round_bf16(synth.act("c3.gate", T * s.top_k, s.ff))
    u = oracle.round_bf16(synth.act("c3.up", T * s.top_k, s.ff))
    h = torch.empty(T * s.top_k, s.ff, device=DEV, dtype=torch.bfloat16)
    ops.silu_mul(to_dev(g, "bf16"), to_dev(u, "bf16"), y=h)
    assert_bf16_within_1ulp(bits16(h), orc.silu_mul(g.copy(), u, threads=THREADS), "routed SwiGLU")
    # fused Q / K per-head norm + RoPE with the step's rotation table: the persistent, shared-memory-staged kernel
    # (the default at this size) against the oracle, and against the direct kernel bit for bit
    q = oracle.round_bf16(synth.act("c5.q", T, s.q_heads, s.head_dim))
    k = oracle.round_bf16(synth.act("c5.k", T, s.kv_heads, s.head_dim))
    wq, wk = synth.norm_w("c5.wq", s.head_dim), synth.norm_w("c5.wk", s.head_dim)
    pos0 = 262144 - T
    tab = ops.rope_table(torch.empty(T, 2, s.rot // 2, device=DEV), s.rot, s.theta, pos0=pos0)
    outs = []
    for staged in (1, 0):
        lib().tune("rope_staged", staged)
        try:
            dq, dk = to_dev(q, "bf16"), to_dev(k, "bf16")
            ops.norm_rope_qk_table(dq, dk, to_dev(wq), to_dev(wk), s.eps, s.rot, tab)
            outs.append((dq, dk))
        finally:
            lib().tune("rope_staged", 1)
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1]), "staged and direct kernels differ"
    pos = np.arange(pos0, pos0 + T, dtype=np.uint32)
    for got, x, w, heads in ((outs[0][0], q, wq, s.q_heads), (outs[0][1], k, wk, s.kv_heads)):
        want = orc.rope_rows(orc.rmsnorm_rows(x.reshape(-1, s.head_dim).copy(), ONE + w, s.eps, threads=THREADS)
                             .reshape(T, heads, s.head_dim), pos, s.rot, s.theta, threads=THREADS)
        assert_bf16_rope(bits16(got), want, "full-size norm + RoPE")


# ---- the gates over their whole argument range ------------------------------------------------------
def gate_arguments():
    """[-104, 89] densely (beyond +-88.7 expf overflows / the sigmoid underflows), the band where the CPU sigmoid is
    subnormal sampled finely, zeros of both signs and infinities."""
    z = np.concatenate([np.linspace(-104.0, 89.0, 193 * 64 + 1), np.linspace(-88.8, -87.2, 2049),
                        np.array([0.0, -0.0, np.inf, -np.inf, 1e-30, -1e-30, 88.72, -88.72])]).astype(np.float32)
    pad = (-z.size) % 1024
    return np.concatenate([z, np.zeros(pad, np.float32)])


def same_or_close(got, want, scale=None):
    """|diff| <= 1e-5 |want| + 1e-30 (the SwiGLU contract); NaN where the CPU gives NaN, infinities equal."""
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan), "NaN positions differ"
    inf = np.isinf(want)
    assert np.array_equal(got[inf], want[inf]), "infinities differ"
    ok = ~(nan | inf)
    ref = np.abs(want[ok]) if scale is None else scale[ok]
    assert np.all(np.abs(got[ok].astype(np.float64) - want[ok]) <= 1e-5 * ref + 1e-30)


def test_gate_sweep_swiglu(orc):
    z = gate_arguments()
    for up in (np.ones_like(z), synth.act("t.gs.up", z.size)):
        with np.errstate(all="ignore"):
            want = orc.silu_mul(z.copy(), up)
        dz = to_dev(z)
        ops.silu_mul(dz, to_dev(up))
        same_or_close(f32(dz), want)


@pytest.mark.parametrize("mode", [0, 1])
def test_gate_sweep_gated_norm(orc, mode):
    z = gate_arguments().reshape(-1, 128)
    o = synth.act("t.gs.o", *z.shape)
    w = synth.gated_w("t.gs.w", 128)
    with np.errstate(all="ignore"):
        want = orc.gated_norm_rows(o.copy(), w, z, 1e-6, mode)
    do = to_dev(o)
    ops.gated_norm(do, to_dev(w), to_dev(z), 1e-6, mode=mode)
    # the fp32 contract of the norms: relative to max(|want|, rms of the row)
    finite = np.where(np.isfinite(want), want, 0.0).astype(np.float64)
    rms = np.sqrt((finite ** 2).mean(axis=1, keepdims=True))
    same_or_close(f32(do), want, scale=np.maximum(np.abs(finite), rms))


def test_gate_sweep_conv_silu(orc):
    """The conv kernel's SiLU: kernel width 1 and unit weights make the op SiLU(x) itself."""
    z = gate_arguments()
    z = z[np.isfinite(z)]
    C = 1024
    z = z[: z.size // C * C].reshape(-1, C)
    w = np.ones((C, 1), np.float32)
    with np.errstate(all="ignore"):
        want = orc.conv_l2norm(z, np.zeros((0, C), np.float32), w, 0, 128, 1e-6)
    out = torch.empty(z.shape, device=DEV)
    ops.conv_l2norm(to_dev(z), torch.zeros(1, device=DEV), to_dev(w), out, l2_channels=0, d=128, eps=1e-6)
    same_or_close(f32(out), want)


# ---- shard invariance of the CUDA chain (one GPU) ---------------------------------------------------
def test_cuda_chain_shards_equal_the_unsharded_run():
    """The op chain run on tokens [b, e) with pos0 = b gives rows [b, e) of the unsharded run bit for bit:
    every op is row-local and a token's rotation depends only on its absolute position. Uneven shards, so
    lean (full-grid) and general (ragged) kernels meet on the same rows. Every shard has more than 148 tokens:
    below that a launch cannot fill the GPU and the add + norm spreads each row over twice the threads, which
    changes the order of the sum of squares (results stay inside 1e-5, but not bit-identical)."""
    s, T = synth.FULL, 1200
    full = chain_mod.LayerChain(s, T, pos0=1000, vocab=4096)
    bounds = [0, 433, 600, 1200]
    shards = []
    for b, e in zip(bounds[:-1], bounds[1:]):
        sh = chain_mod.LayerChain(s, e - b, pos0=1000 + b, vocab=4096)
        k = max(s.top_k, 1)
        per_token = {"delta_a": 1, "delta_b": 1, "qk": 1, "o": s.v_heads, "z": s.v_heads, "y": s.v_heads, "q": 1, "k": 1,
                     "gate_s": 1, "up_s": 1, "gate_r": k, "up_r": k}
        for bo_s, bo_f in zip(sh.sets, full.sets):
            for name, rows in per_token.items():
                getattr(bo_s, name).copy_(getattr(bo_f, name)[b * rows:e * rows])
        sh.table.copy_(full.table)
        sh.ids.copy_(full.ids[b:e])
        for attr in ("w_attn", "w_post"):
            for ws, wf in zip(getattr(sh, attr), getattr(full, attr)):
                ws.copy_(wf)
        for attr in ("w_q", "w_k", "w_gated"):
            getattr(sh, attr).copy_(getattr(full, attr))
        shards.append((b, e, sh, per_token))
    full.step()
    for b, e, sh, per_token in shards:
        sh.step()
        torch.cuda.synchronize()
        assert torch.equal(sh.res, full.res[b:e]), f"residual of shard [{b}, {e})"
        assert torch.equal(sh.xn, full.xn[b:e]), f"xn of shard [{b}, {e})"
        assert torch.equal(sh.h_s, full.h_s[b:e]) and torch.equal(sh.h_r, full.h_r[b * s.top_k:e * s.top_k])
        for bo_s, bo_f in zip(sh.sets, full.sets):
            for name in ("qk", "y", "q", "k"):
                rows = per_token[name]
                assert torch.equal(getattr(bo_s, name), getattr(bo_f, name)[b * rows:e * rows]), f"{name} of shard [{b}, {e})"


# ---- negative controls: the tolerances reject the reference's planted mutants ------------------------
def test_l2_norm_is_not_an_rms_norm(orc):
    """k-l2norm-as-rms (tests/mutants.toml:312-320): eps is added to the SUM of squares. Rows of small norm make the
    two recipes differ by far more than 1e-5; the CUDA result must match the true one and fail the mutant."""
    rows, d, eps = 64, 128, 1e-6
    x = (synth.act("t.nc.l2", rows, d) * np.float32(1e-3)).astype(np.float32)
    dx = to_dev(x)
    ops.l2norm(dx, eps)
    got = f32(dx)
    assert_rows_close(got, orc.l2norm_rows(x.copy(), eps), what="l2norm, small rows")
    ss = (x.astype(np.float64) ** 2).sum(axis=1, keepdims=True)
    mutant = (x / np.sqrt(ss / d + eps)).astype(np.float32)
    with pytest.raises(AssertionError):
        assert_rows_close(got, mutant, what="mutant k-l2norm-as-rms")
    mean_eps = (x / np.sqrt(ss + eps * d)).astype(np.float32)  # eps inside a mean, rescaled
    with pytest.raises(AssertionError):
        assert_rows_close(got, mean_eps, what="mutant eps-inside-the-mean")


def test_rope_rotation_direction(orc):
    """k-rope-sign (tests/mutants.toml:288-296): v[i] = a c + b s instead of a c - b s."""
    s, T = synth.FULL, 16
    x = synth.act("t.nc.rope", T, s.q_heads, s.head_dim)
    pos = synth.positions("t.nc.pos", T, s.max_pos)
    dx = to_dev(x)
    ops.rope(dx, None, s.rot, s.theta, params=to_dev(pos.view(np.int32)), pstride=1)
    got = f32(dx)
    half = s.rot // 2

    def check(want):
        bound = 1e-5 * np.maximum(np.maximum(np.abs(x[..., :half]), np.abs(x[..., half:s.rot])), 1e-30)
        assert np.all(np.abs(got[..., :half] - want[..., :half]) <= bound)
        assert np.all(np.abs(got[..., half:s.rot] - want[..., half:s.rot]) <= bound)

    check(orc.rope_rows(x.copy(), pos, s.rot, s.theta))
    inv = orc.rope_inv_freq(s.rot, s.theta)
    ang = pos.astype(np.float32)[:, None] * inv[None, :]
    c, sn = np.cos(ang.astype(np.float64))[:, None, :], np.sin(ang.astype(np.float64))[:, None, :]
    mutant = x.copy()
    mutant[..., :half] = x[..., :half] * c + x[..., half:s.rot] * sn
    mutant[..., half:s.rot] = x[..., :half] * sn + x[..., half:s.rot] * c
    with pytest.raises(AssertionError):
        check(mutant)


def test_scale_silu_applies_its_scale(orc):
    """k-scale-silu-scale (tests/mutants.toml:228-236): Silu(x) instead of Silu(x * scale)."""
    n, scale = 4096, 0.25
    x = (synth.act("t.nc.ss", n) * 4).astype(np.float32)
    dx = to_dev(x)
    st = torch.cuda.current_stream().cuda_stream
    lib().call("scale_silu", st, dx.data_ptr(), dx.data_ptr(), 0, scale, n)
    got = f32(dx)
    true = np.array([orc._call("orc_silu", float(np.float32(v) * np.float32(scale))) for v in x], np.float32)
    mutant = np.array([orc._call("orc_silu", float(v)) for v in x], np.float32)
    assert np.all(np.abs(got - true) <= 1e-5 * np.abs(true) + 1e-30)
    assert not np.all(np.abs(got - mutant) <= 1e-5 * np.abs(mutant) + 1e-30)
