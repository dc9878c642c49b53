"""Parity of the CUDA kernels with the CPU oracle, through the C ABI (GPU only).

Tolerances (the contract of the path): embedding gather / dequant, RoPE position
selection, residual sums and Q8 codes bit-exact; fp32 outputs within 1e-5 relative
(per-row rel-L2 and per-element against max(|want|, row rms)); bf16 outputs within
1 bf16 ulp of bf16_rne(oracle fp32). Every output buffer is surrounded by
NaN-poisoned guard regions, so a write outside the tensor fails the test.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_bf16_rope, assert_bf16_within_1ulp, assert_rows_close
from halo_flash_b200 import HaloError, lib, ops, synth

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
ONE = np.float32(1.0)
GUARD = 64  # elements of poison on each side of a guarded buffer


# ---- device helpers ----------------------------------------------------------------
def to_dev(a: np.ndarray, dtype=None) -> torch.Tensor:
    """numpy -> CUDA tensor; dtype 'bf16' / 'f16' rounds to nearest even first."""
    if dtype == "bf16":
        return torch.from_numpy(oracle.bf16_bits(a).view(np.int16)).to(DEV).view(torch.bfloat16).reshape(a.shape)
    if dtype == "f16":
        return torch.from_numpy(a.astype(np.float16)).to(DEV)
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def to_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


class Guarded:
    """An output tensor inside a larger allocation whose margins hold a poison pattern."""

    def __init__(self, shape, dtype, offset_elems=0):
        n = int(np.prod(shape))
        self.raw = torch.empty(n + 2 * GUARD + offset_elems, dtype=dtype, device=DEV)
        self.poison = float("nan") if dtype.is_floating_point else 0x7F
        self.raw.fill_(self.poison)
        self.lo = GUARD + offset_elems
        self.t = self.raw[self.lo:self.lo + n].view(shape)
        self.n = n

    def check(self, what=""):
        for part in (self.raw[:self.lo], self.raw[self.lo + self.n:]):
            if isinstance(self.poison, int):
                assert bool((part == self.poison).all()), f"{what}: write outside the output buffer"
            else:
                assert bool(torch.isnan(part.float()).all()), f"{what}: write outside the output buffer"


def rounded(a, dtype):
    if dtype == "bf16":
        return oracle.round_bf16(a)
    if dtype == "f16":
        return a.astype(np.float16).astype(np.float32)
    return a


TDT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def check_out(t: torch.Tensor, want: np.ndarray, what: str):
    """Compare a device tensor with the oracle's fp32 result at the tensor's precision."""
    if t.dtype == torch.float32:
        assert_rows_close(to_f32(t), want, what=what)
    elif t.dtype == torch.bfloat16:
        assert_bf16_within_1ulp(bits16(t), want, what=what)
    else:  # fp16: within 1 fp16 ulp of half_rne(want)
        got = bits16(t).astype(np.int32)
        ref = want.astype(np.float16).view(np.uint16).astype(np.int32)
        order = lambda b: np.where(b & 0x8000, 0x8000 - (b & 0x7FFF) - 1, 0x8000 + b)
        assert np.abs(order(got.reshape(-1)) - order(ref.reshape(-1))).max() <= 1, what


# ---- golden fixtures produced by the reference's own CPU code ---------------------------
def test_golden_tiny_chain(golden_ops):
    gd, s = golden_ops, synth.C1
    res, delta = to_dev(gd["res"]), to_dev(gd["delta"])
    xn = Guarded(gd["xn"].shape, torch.float32)
    q8 = Guarded(gd["xn_q8_0"].shape, torch.uint8)
    ops.add_rmsnorm(res, delta, to_dev(gd["norm_w"]), s.eps, one_plus=True, xn=xn.t, q8_0=q8.t)
    assert to_f32(res).tobytes() == gd["res_out"].tobytes()
    assert_rows_close(to_f32(xn.t), gd["xn"], what="add_rmsnorm")
    xn.check("xn"), q8.check("q8")
    qk = to_dev(gd["qk"])
    ops.l2norm(qk, s.eps)
    assert_rows_close(to_f32(qk), gd["qk_l2"], what="l2norm")
    for mode, key in ((0, "gated_silu"), (1, "gated_sigmoid")):
        o = to_dev(gd["o"])
        ops.gated_norm(o, to_dev(gd["gated_w"]), to_dev(gd["z"]), s.eps, mode=mode)
        assert_rows_close(to_f32(o), gd[key], what=key)
    q, k = to_dev(gd["q"]), to_dev(gd["k"])
    pos = to_dev(gd["pos"].view(np.int32))
    used = torch.zeros(32, dtype=torch.int32, device=DEV)
    ops.rope(q, k, s.rot, s.theta, params=pos, pstride=1, pos_out=used)
    assert np.array_equal(used.cpu().numpy().view(np.uint32), gd["pos"])
    check_rope(to_f32(q), gd["q_rope"], gd["q"], s.rot, "q rope")
    check_rope(to_f32(k), gd["k_rope"], gd["k"], s.rot, "k rope")
    qn = to_dev(gd["q"]).view(-1, s.head_dim)
    ops.norm_rope(qn, to_dev(gd["qnorm_w"]), s.eps, s.rot, s.theta, s.q_heads, params=pos, pstride=1)
    assert_rows_close(to_f32(qn), gd["q_norm_rope"].reshape(-1, s.head_dim), what="norm_rope")
    g = to_dev(gd["gate"])
    ops.silu_mul(g, to_dev(gd["up"]))
    assert_rows_close(to_f32(g), gd["swiglu"], what="swiglu")
    table = np.zeros((s.vocab, s.q8_row_bytes), np.uint8)
    table[gd["table_rows"]] = gd["table_bytes"]
    out = Guarded(gd["embed"].shape, torch.float32)
    ops.embed_q8_0(to_dev(table), to_dev(gd["ids"].view(np.int32)), s.hidden, out.t)
    assert to_f32(out.t).tobytes() == gd["embed"].tobytes()
    out.check("embed")


def check_rope(got, want, x_in, rot, what):
    """|diff| <= 1e-5 * max(|a|, |b|) per rotated pair; dims >= rot untouched bit for bit."""
    half = rot // 2
    a, b = np.abs(x_in[..., :half]), np.abs(x_in[..., half:rot])
    bound = 1e-5 * np.maximum(np.maximum(a, b), 1e-30)
    assert np.all(np.abs(got[..., :half] - want[..., :half]) <= bound), what
    assert np.all(np.abs(got[..., half:rot] - want[..., half:rot]) <= bound), what
    assert got[..., rot:].tobytes() == x_in[..., rot:].tobytes(), what + " (dims beyond rot changed)"


# ---- group 1 ---------------------------------------------------------------------------
@pytest.mark.parametrize("rows,d", [(1, 256), (3, 256), (32, 256), (5, 2048), (4, 2560), (3, 4096), (2, 8200),
                                    (7, 100), (9, 8), (2, 16384)])
@pytest.mark.parametrize("one_plus", [True, False])
def test_add_rmsnorm_fp32(orc, rows, d, one_plus):
    res, delta, w = synth.act("t.res", rows, d), synth.act("t.delta", rows, d), synth.norm_w("t.w", d)
    g = ONE + w if one_plus else w
    summed = res + delta
    want = orc.rmsnorm_rows(summed.copy(), g, 1e-6)
    dres = to_dev(res)
    xn = Guarded((rows, d), torch.float32)
    ops.add_rmsnorm(dres, to_dev(delta), to_dev(w), 1e-6, one_plus=one_plus, xn=xn.t)
    assert to_f32(dres).tobytes() == summed.tobytes(), "residual sum must be the single fp32 add"
    assert_rows_close(to_f32(xn.t), want, what=f"add_rmsnorm {rows}x{d}")
    xn.check()


# 2560 = 5 x 64 octets, 3072 = 3 x 128, 1536 = 3 x 64, 5120 = 5 x 128: launches of whole CTAs of such rows that can fill
# the GPU take the lean kernel with three or five octets per thread, shorter or ragged ones the general kernel
@pytest.mark.parametrize("rows,d", [(1, 2048), (8, 2048), (33, 2048), (5, 256), (3, 2560), (6, 104), (128, 2560), (8, 2560),
                                    (128, 3072), (256, 1536), (64, 5120)])
@pytest.mark.parametrize("xn_dtype", ["bf16", "f32"])
def test_add_rmsnorm_bf16_residual(orc, rows, d, xn_dtype):
    res = rounded(synth.act("t.res", rows, d) * 3, "bf16")
    delta = rounded(synth.act("t.delta", rows, d), "bf16")
    w = synth.norm_w("t.w", d)
    stored = oracle.round_bf16(res + delta)  # one add, one rounding; the norm reads this
    want = orc.rmsnorm_rows(stored.copy(), ONE + w, 1e-6)
    dres = to_dev(res, "bf16")
    xn = Guarded((rows, d), TDT[xn_dtype])
    ops.add_rmsnorm(dres, to_dev(delta, "bf16"), to_dev(w), 1e-6, xn=xn.t)
    assert np.array_equal(bits16(dres), oracle.bf16_bits(stored)), "stored residual must be bf16_rne(res + delta)"
    check_out(xn.t, want, f"xn {xn_dtype}")
    xn.check()


@pytest.mark.parametrize("rows,d,res_dtype", [(4, 256, "f32"), (8, 2048, "bf16"), (3, 2560, "f32"), (5, 96, "f32"),
                                              (2, 4096, "bf16"), (128, 2560, "bf16"), (128, 3072, "bf16"), (256, 1536, "f32")])
def test_q8_epilogues_two_stage(orc, rows, d, res_dtype):
    """Stage 1: the fp32 xn matches the oracle within 1e-5. Stage 2: the Q8_0 blocks and the
    int8 + fp32-scale form equal the oracle's encoders applied to the GPU's own xn, bit for
    bit (the reference's rule, tests/gpu/quant_gpu_test.cpp:2428-2494)."""
    res = rounded(synth.act("t.q.res", rows, d) * 2, res_dtype)
    delta = rounded(synth.act("t.q.delta", rows, d), res_dtype)
    res[0, :32] = 0  # a block whose scale is zero
    delta[0, :32] = 0
    w = synth.norm_w("t.q.w", d)
    stored = rounded(res + delta, res_dtype)
    want = orc.rmsnorm_rows(stored.copy(), ONE + w, 1e-6)
    dt = None if res_dtype == "f32" else res_dtype
    xn = Guarded((rows, d), torch.float32)
    q8 = Guarded((rows, d // 32 * 34), torch.uint8)
    xq, xd = Guarded((rows, d), torch.int8), Guarded((rows, d // 32), torch.float32)
    ops.add_rmsnorm(to_dev(res, dt), to_dev(delta, dt), to_dev(w), 1e-6, xn=xn.t, q8_0=q8.t, xq=xq.t, xd=xd.t)
    own = to_f32(xn.t)
    assert_rows_close(own, want, what="xn")
    assert q8.t.cpu().numpy().tobytes() == orc.encode_q8_0_rows(own).tobytes(), "Q8_0 blocks"
    wq, wd = orc.quantize_i8_rows(own)
    assert xq.t.cpu().numpy().tobytes() == wq.tobytes() and to_f32(xd.t).tobytes() == wd.tobytes(), "int8 form"
    for gd in (xn, q8, xq, xd):
        gd.check()
    # Q8_0 as the only output: identical bytes
    q8b = Guarded((rows, d // 32 * 34), torch.uint8)
    ops.add_rmsnorm(to_dev(res, dt), to_dev(delta, dt), to_dev(w), 1e-6, q8_0=q8b.t)
    assert torch.equal(q8b.t, q8.t)
    q8b.check()


@pytest.mark.parametrize("xdt,ydt", [("f32", "f32"), ("bf16", "f32"), ("f16", "f32"), ("bf16", "bf16"),
                                     ("f32", "bf16"), ("f16", "f16")])
def test_rmsnorm_dtypes_and_gamma_rows(orc, xdt, ydt):
    """Grouped gammas: row r uses (r % w_period) * w_stride (src/kernels/core.hip:4049)."""
    rows, d, period = 10, 512, 4
    x = rounded(synth.act("t.rn.x", rows, d), xdt)
    w = synth.gated_w("t.rn.w", period * d).reshape(period, d)
    want = orc.rmsnorm_rows(x.copy(), w, 1e-6, w_stride=d, w_period=period)
    y = Guarded((rows, d), TDT[ydt])
    ops.rmsnorm(to_dev(x, None if xdt == "f32" else xdt), to_dev(w), 1e-6, y=y.t, w_stride=d, w_period=period)
    check_out(y.t, want, f"{xdt}->{ydt}")
    y.check()


def test_rmsnorm_in_place_unaligned_and_strided(orc):
    d, rows = 256, 6
    x, w = synth.act("t.ip.x", rows, d), synth.gated_w("t.ip.w", d)
    want = orc.rmsnorm_rows(x.copy(), w, 1e-6)
    dx = to_dev(x)
    ops.rmsnorm(dx, to_dev(w), 1e-6)
    assert_rows_close(to_f32(dx), want, what="in place")
    # 4-byte-aligned (not 16) views take the scalar kernel and must agree
    buf = Guarded((rows, d), torch.float32, offset_elems=1)
    buf.t.copy_(to_dev(x))
    ops.rmsnorm(buf.t, to_dev(w), 1e-6)
    assert_rows_close(to_f32(buf.t), want, what="unaligned")
    buf.check()
    # per-entry strides of the batched-decode form (halo_rmsnorm_y): entry e at x + e * stride
    nvec, batch, stride = 2, 3, 2 * d + 64
    arena = synth.act("t.ip.arena", batch * stride)
    w2 = synth.gated_w("t.ip.w2", nvec * d).reshape(nvec, d)
    darena = to_dev(arena)
    dw2 = to_dev(w2)
    lib().call("rmsnorm_y", torch.cuda.current_stream().cuda_stream, darena.data_ptr(), dw2.data_ptr(), d, 1e-6,
               d, stride, nvec, batch)
    got = to_f32(darena)
    for e in range(batch):
        rows_e = arena[e * stride:e * stride + nvec * d].reshape(nvec, d).copy()
        want_e = orc.rmsnorm_rows(rows_e, w2, 1e-6, w_stride=d, w_period=nvec)
        assert_rows_close(got[e * stride:e * stride + nvec * d].reshape(nvec, d), want_e, what=f"entry {e}")
        tail = slice(e * stride + nvec * d, (e + 1) * stride)
        assert got[tail].tobytes() == arena[tail].tobytes(), "bytes between entries must stay untouched"


def test_rmsnorm_rows_h_fp16_copy(orc):
    """fp32 y within tolerance; the fp16 copy is half_rne(y) bit for bit, row-major and K-blocked
    (tests/gpu/quant_gpu_test.cpp:2361-2422)."""
    T, hc, d = 5, 4, 128
    x, w = synth.act("t.h.x", T * hc, d), synth.gated_w("t.h.w", hc * d).reshape(hc, d)
    want = orc.rmsnorm_rows(x.copy(), w, 1e-6, w_stride=d, w_period=hc)
    s = torch.cuda.current_stream().cuda_stream
    dx, dw = to_dev(x), to_dev(w)
    for tokens in (0, T):
        y = Guarded((T * hc, d), torch.float32)
        y16 = Guarded((T * hc, d), torch.float16)
        lib().call("rmsnorm_rows_h", s, dx.data_ptr(), 0, dw.data_ptr(), y.t.data_ptr(), y16.t.data_ptr(),
                   d, 1e-6, d, hc, None, None, 0, tokens, T * hc)
        got = to_f32(y.t)
        assert_rows_close(got, want, what="y")
        h = y16.t.cpu().numpy().reshape(-1)
        exp = got.astype(np.float16)
        if tokens:  # [cols / 64][T][64] with cols = hc * d
            blocked = exp.reshape(T, hc * d // 64, 64).transpose(1, 0, 2).reshape(-1)
            assert h.tobytes() == blocked.tobytes()
        else:
            assert h.tobytes() == exp.reshape(-1).tobytes()
        y.check(), y16.check()


# ---- group 2 ---------------------------------------------------------------------------
@pytest.mark.parametrize("rows,d", [(8, 64), (64, 128), (33, 128), (5, 100), (3, 1024)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_l2norm(orc, rows, d, dtype):
    x = rounded(synth.act("t.l2.x", rows, d) * 0.3, dtype)
    want = orc.l2norm_rows(x.copy(), 1e-6)
    dx = to_dev(x, None if dtype == "f32" else dtype)
    ops.l2norm(dx, 1e-6)
    check_out(dx, want, f"l2norm {dtype}")
    z = torch.zeros(4, 128, device=DEV)
    ops.l2norm(z, 1e-6)
    assert not z.any()  # eps keeps an all-zero head finite


@pytest.mark.parametrize("odt,zdt,ydt", [("f32", "f32", "f32"), ("f32", "f32", "f16"), ("f32", "f16", "f16"),
                                         ("f16", "f16", "f16"), ("bf16", "bf16", "bf16"), ("bf16", "bf16", "f32"),
                                         ("f32", "f32", "bf16")])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("rows,d", [(16, 64), (96, 128), (7, 100)])
def test_gated_norm(orc, odt, zdt, ydt, mode, rows, d):
    o = rounded(synth.act("t.gn.o", rows, d) * 2, odt)
    z = rounded(synth.act("t.gn.z", rows, d) * 3, zdt)
    w = synth.gated_w("t.gn.w", d)
    want = orc.gated_norm_rows(o.copy(), w, z, 1e-6, mode)
    y = Guarded((rows, d), TDT[ydt])
    ops.gated_norm(to_dev(o, None if odt == "f32" else odt), to_dev(w), to_dev(z, None if zdt == "f32" else zdt), 1e-6,
                   mode=mode, y=y.t)
    check_out(y.t, want, f"gated {odt},{zdt}->{ydt} mode {mode}")
    y.check()


def test_gated_norm_rejects_unsupported_dtype_mix():
    o = torch.zeros(4, 128, device=DEV, dtype=torch.float16)
    z = torch.zeros(4, 128, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(HaloError, match="dtype combination"):
        ops.gated_norm(o, torch.ones(128, device=DEV), z, 1e-6)


# ---- group 3 ---------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [synth.C1, synth.FULL])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_rope_q_and_k_random_positions(orc, shape, dtype):
    s, T = shape, 19
    q = rounded(synth.act("t.r.q", T, s.q_heads, s.head_dim), dtype)
    k = rounded(synth.act("t.r.k", T, s.kv_heads, s.head_dim), dtype)
    pos = synth.positions("t.r.pos", T, s.max_pos)
    pos[0], pos[1] = 0, s.max_pos - 1
    wq, wk = orc.rope_rows(q.copy(), pos, s.rot, s.theta), orc.rope_rows(k.copy(), pos, s.rot, s.theta)
    dt = None if dtype == "f32" else dtype
    dq, dk = to_dev(q, dt), to_dev(k, dt)
    used = Guarded((T,), torch.int32)
    # positions live in parameter rows 16 uint32 apart, slot 1 (kHaloPosition)
    params = np.zeros((T, 16), np.uint32)
    params[:, 1] = pos
    ops.rope(dq, dk, s.rot, s.theta, params=to_dev(params.view(np.int32)), pstride=16, slot=1, pos_out=used.t)
    assert np.array_equal(used.t.cpu().numpy().view(np.uint32), pos), "position selection must be exact"
    used.check()
    if dtype == "f32":
        check_rope(to_f32(dq), wq, q, s.rot, "q")
        check_rope(to_f32(dk), wk, k, s.rot, "k")
    else:
        assert_bf16_rope(bits16(dq), wq, "q bf16")
        assert_bf16_rope(bits16(dk), wk, "k bf16")
        assert np.array_equal(bits16(dq)[..., s.rot:], oracle.bf16_bits(q)[..., s.rot:])


def test_rope_position_forms(orc):
    """pos0 + t (halo_rope_neox_rows), params[slot] * scale (halo_rope_neox_p), (b0 + b) * ratio
    (halo_rope_neox_blocks), per-entry params (halo_rope_neox_p_y): src/kernels/core.hip:289-311."""
    s = synth.FULL
    st = torch.cuda.current_stream().cuda_stream
    heads, hd, rot, T = 3, s.head_dim, s.rot, 6
    x = synth.act("t.rp.x", T, heads, hd)
    # rows: pos0 + t, up to the largest position of the decode configuration
    pos0 = 262144 - T
    dx = to_dev(x)
    lib().call("rope_neox_rows", st, dx.data_ptr(), hd, rot, pos0, heads, s.theta, T * heads)
    check_rope(to_f32(dx), orc.rope_rows(x.copy(), np.arange(pos0, pos0 + T, dtype=np.uint32), rot, s.theta), x, rot,
               "rows")
    # single position for every head
    dx = to_dev(x[:1])
    lib().call("rope_neox", st, dx.data_ptr(), hd, rot, 300000, s.theta, heads)
    check_rope(to_f32(dx), orc.rope_rows(x[:1].copy(), np.array([300000], np.uint32), rot, s.theta), x[:1], rot, "one")
    # params[slot] * scale
    params = to_dev(np.array([7, 4097, 9, 11], np.uint32).view(np.int32))
    dx = to_dev(x[:1])
    lib().call("rope_neox_p", st, dx.data_ptr(), params.data_ptr(), hd, rot, 1, 4, s.theta, heads)
    check_rope(to_f32(dx), orc.rope_rows(x[:1].copy(), np.array([4097 * 4], np.uint32), rot, s.theta), x[:1], rot, "p")
    # pooled blocks: one head-sized row per block at (b0 + b) * ratio
    blocks = synth.act("t.rp.b", 5, 1, hd)
    dx = to_dev(blocks)
    lib().call("rope_neox_blocks", st, dx.data_ptr(), hd, rot, 10, 128, s.theta, 5)
    check_rope(to_f32(dx), orc.rope_rows(blocks.copy(), (np.arange(10, 15) * 128).astype(np.uint32), rot, s.theta),
               blocks, rot, "blocks")
    # per-entry: entry e at x + e * stride with params + e * pstride
    B, stride, pstride = 4, heads * hd + 32, 16
    arena = synth.act("t.rp.arena", B * stride)
    prm = np.zeros((B, pstride), np.uint32)
    prm[:, 1] = [5, 99999, 0, 262143]
    darena = to_dev(arena)
    dprm = to_dev(prm.view(np.int32))
    lib().call("rope_neox_p_y", st, darena.data_ptr(), dprm.data_ptr(), hd, rot, 1, 1, s.theta,
               stride, pstride, heads, B)
    got = to_f32(darena)
    for e in range(B):
        xe = arena[e * stride:e * stride + heads * hd].reshape(1, heads, hd)
        check_rope(got[e * stride:e * stride + heads * hd].reshape(1, heads, hd),
                   orc.rope_rows(xe.copy(), prm[e:e + 1, 1], rot, s.theta), xe, rot, f"entry {e}")
        assert got[e * stride + heads * hd:(e + 1) * stride].tobytes() == arena[e * stride + heads * hd:(e + 1) * stride].tobytes()


def test_rope_scalar_path_odd_rotary_dim(orc):
    heads, hd, rot, T = 2, 24, 6, 5
    x = synth.act("t.rs.x", T, heads, hd)
    pos = np.array([0, 1, 17, 4095, 100000], np.uint32)
    dx = to_dev(x)
    ops.rope(dx, None, rot, 5e5, params=to_dev(pos.view(np.int32)), pstride=1)
    check_rope(to_f32(dx), orc.rope_rows(x.copy(), pos, rot, 5e5), x, rot, "scalar rope")


@pytest.mark.parametrize("shape", [synth.C1, synth.FULL])
@pytest.mark.parametrize("T", [9, 64])
def test_fused_norm_rope_equals_separate_kernels_and_oracle(orc, shape, T):
    """Fused per-head RMSNorm + RoPE vs the separate kernels bit for bit (the reference's
    NormRopeEqualsSeparateKernels / SplitQgateNormRopeEqualsSeparateKernels,
    tests/gpu/quant_gpu_test.cpp:2635-2749, pos0 up to 300000) and vs the oracle. T = 9 leaves ragged CTAs
    (the general kernels), T = 64 fills them (the lean ones)."""
    s, pos0 = shape, 299990
    heads, hd = s.q_heads, s.head_dim
    qg = synth.act("t.f.qg", T * heads, 2 * hd)
    w = synth.norm_w("t.f.w", hd)
    st = torch.cuda.current_stream().cuda_stream
    # separate: split, per-head norm (1 + w folded on the host, as the GGUF stores it), rope
    g = ONE + w
    q1, gate1 = torch.empty(T * heads, hd, device=DEV), torch.empty(T * heads, hd, device=DEV)
    dqg, dg = to_dev(qg), to_dev(g)
    lib().call("split_qgate", st, dqg.data_ptr(), q1.data_ptr(), gate1.data_ptr(), hd, T * heads)
    lib().call("rmsnorm", st, q1.data_ptr(), dg.data_ptr(), q1.data_ptr(), hd, s.eps, 0, T * heads)
    lib().call("rope_neox_rows", st, q1.data_ptr(), hd, s.rot, pos0, heads, s.theta, T * heads)
    # fused
    q2, gate2 = Guarded((T * heads, hd), torch.float32), Guarded((T * heads, hd), torch.float32)
    lib().call("split_qgate_norm_rope", st, dqg.data_ptr(), q2.t.data_ptr(), gate2.t.data_ptr(),
               dg.data_ptr(), s.eps, s.rot, pos0, heads, s.theta, hd, T * heads)
    assert torch.equal(gate1, gate2.t) and to_f32(gate1).tobytes() == qg[:, hd:].tobytes()
    assert torch.equal(q1, q2.t), "fused kernel must equal the three separate kernels bit for bit"
    q2.check(), gate2.check()
    want = orc.rmsnorm_rows(np.ascontiguousarray(qg[:, :hd]), g, s.eps)
    want = orc.rope_rows(want.reshape(T, heads, hd), np.arange(pos0, pos0 + T, dtype=np.uint32), s.rot, s.theta)
    assert_rows_close(to_f32(q2.t), want.reshape(-1, hd), what="fused vs oracle")
    # in place on K rows with the cache append, one_plus applied on the device
    k = synth.act("t.f.k", T * s.kv_heads, hd)
    dk, cache = to_dev(k), Guarded((T * s.kv_heads, hd), torch.float32)
    ops.norm_rope(dk, to_dev(w), s.eps, s.rot, s.theta, s.kv_heads, cache=cache.t, one_plus=True, pos0=pos0)
    wantk = orc.rope_rows(orc.rmsnorm_rows(k.copy(), g, s.eps).reshape(T, s.kv_heads, hd),
                          np.arange(pos0, pos0 + T, dtype=np.uint32), s.rot, s.theta)
    assert_rows_close(to_f32(dk), wantk.reshape(-1, hd), what="k norm+rope")
    assert torch.equal(dk, cache.t)
    cache.check()


def test_fused_norm_rope_bf16(orc):
    s, T = synth.FULL, 7
    heads, hd = s.q_heads + s.kv_heads, s.head_dim
    x = rounded(synth.act("t.fb.x", T * heads, hd), "bf16")
    w = synth.norm_w("t.fb.w", hd)
    pos = synth.positions("t.fb.pos", T, s.max_pos)
    want = orc.rope_rows(orc.rmsnorm_rows(x.copy(), ONE + w, s.eps).reshape(T, heads, hd), pos, s.rot, s.theta)
    dx = to_dev(x, "bf16")
    ops.norm_rope(dx, to_dev(w), s.eps, s.rot, s.theta, heads, params=to_dev(pos.view(np.int32)), pstride=1)
    assert_bf16_rope(bits16(dx), want.reshape(-1, hd), "norm_rope bf16")


# ---- group 4 ---------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 7, 8, 128, 4099, 65536 + 3, 10 * 512 * 33])
@pytest.mark.parametrize("idt,ydt", [("f32", "f32"), ("f32", "f16"), ("f32", "bf16"), ("bf16", "bf16"), ("f16", "f16"),
                                     ("bf16", "f32")])
def test_silu_mul(orc, n, idt, ydt):
    g = rounded(synth.act("t.s.g", n) * 4, idt)
    up = rounded(synth.act("t.s.up", n), idt)
    want = orc.silu_mul(g.copy(), up)
    y = Guarded((n,), TDT[ydt])
    dt = None if idt == "f32" else idt
    ops.silu_mul(to_dev(g, dt), to_dev(up, dt), y=y.t)
    got = y.t
    if ydt == "f32":
        gotf = to_f32(got).astype(np.float64)
        assert np.all(np.abs(gotf - want) <= 1e-5 * np.abs(want) + 1e-30), "swiglu rel 1e-5 elementwise"
    else:
        check_out(got.view(1, -1), want.reshape(1, -1), f"swiglu {ydt}")
    y.check()


def test_silu_mul_in_place_and_unaligned(orc):
    n = 1000
    g, up = synth.act("t.si.g", n) * 5, synth.act("t.si.up", n)
    want = orc.silu_mul(g.copy(), up)
    buf = Guarded((n,), torch.float32, offset_elems=3)
    buf.t.copy_(to_dev(g))
    ops.silu_mul(buf.t, to_dev(up))
    gotf = to_f32(buf.t).astype(np.float64)
    assert np.all(np.abs(gotf - want) <= 1e-5 * np.abs(want) + 1e-30)
    buf.check()
    # extreme arguments: saturated sigmoid on both sides
    ext = np.array([-100.0, -20.0, -1e-3, 0.0, 1e-3, 20.0, 100.0, 3.0], np.float32)
    d = to_dev(ext)
    ops.silu_mul(d, to_dev(np.ones(8, np.float32)))
    wante = orc.silu_mul(ext.copy(), np.ones(8, np.float32))
    assert np.all(np.abs(to_f32(d) - wante) <= 1e-5 * np.abs(wante) + 1e-37)


# ---- group 5 ---------------------------------------------------------------------------
@pytest.mark.parametrize("vocab,cols,T", [(4096, 256, 32), (1000, 2048, 77), (64, 32, 9), (300, 96, 40)])
@pytest.mark.parametrize("odt", ["f32", "bf16"])
def test_embedding_gather_bit_exact(orc, vocab, cols, T, odt):
    """cols 32 / 96 have 34 / 102-byte rows (not 16-byte multiples): the byte-load kernel."""
    table = synth.q8_0_table("t.e.table", vocab, cols)
    ids = synth.token_ids("t.e.ids", T, vocab)
    ids[0], ids[-1] = 0, vocab - 1
    want = orc.embed_q8_0_rows(table, ids, cols)
    out = Guarded((T, cols), TDT[odt])
    ops.embed_q8_0(to_dev(table), to_dev(ids.view(np.int32)), cols, out.t)
    if odt == "f32":
        assert to_f32(out.t).tobytes() == want.tobytes()
    else:
        assert np.array_equal(bits16(out.t), oracle.bf16_bits(want))
    out.check()


@pytest.mark.parametrize("cols", [1024, 2048, 2560])
@pytest.mark.parametrize("odt", ["f32", "bf16", "f16"])
def test_embedding_long_launches_read_rows_directly(orc, cols, odt):
    """Launches with more rows than resident warps read rows straight into registers (rows of 32, 64 and 80 blocks have
    direct kernels): the result equals the shared-memory-staged kernel's bit for bit, the oracle's on a sample of rows,
    and out-of-range ids give zero rows. The table's last row is among the ids: its last block ends the allocation."""
    vocab, T = 3000, 5000
    table = synth.q8_0_table("t.ed.table", vocab, cols)
    ids = synth.token_ids("t.ed.ids", T, vocab)
    ids[0], ids[1], ids[-1], ids[7] = 0, vocab - 1, vocab - 1, vocab + 5
    dtab, dids = to_dev(table), to_dev(ids.view(np.int32))
    outs = []
    for direct in (1, 0):
        lib().tune("embed_direct", direct)
        try:
            out = Guarded((T, cols), TDT[odt])
            ops.embed_q8_0(dtab, dids, cols, out.t, vocab=vocab)
            out.check()
            outs.append(out.t)
        finally:
            lib().tune("embed_direct", 1)
    assert torch.equal(outs[0], outs[1])
    assert not outs[0][7].any()
    pick = np.array([0, 1, 2, 100, 2500, T - 1])
    want = orc.embed_q8_0_rows(table, ids[pick], cols)
    got = outs[0][torch.as_tensor(pick, device=DEV)]
    if odt == "f32":
        assert to_f32(got).tobytes() == want.tobytes()
    elif odt == "bf16":
        assert np.array_equal(bits16(got), oracle.bf16_bits(want))
    else:
        assert np.array_equal(got.cpu().numpy().view(np.uint16), want.astype(np.float16).view(np.uint16))


def test_embedding_reference_entry_points(orc):
    """_embed (scalar token), _embed_p (params[kHaloToken]) and _embed_rows (params[t * 16]):
    src/kernels/core.hip:219-232."""
    s = synth.C1
    table = synth.q8_0_table("t.e2.table", 512, s.hidden)
    dtab = to_dev(table)
    st = torch.cuda.current_stream().cuda_stream
    T = 12
    ids = synth.token_ids("t.e2.ids", T, 512)
    params = np.full((T, 16), 0xDEAD, np.uint32)
    params[:, 0] = ids
    dpar = to_dev(params.view(np.int32))
    want = orc.embed_q8_0_rows(table, ids, s.hidden)
    out = Guarded((T, s.hidden), torch.float32)
    lib().call("matvec_q8_0_embed_rows", st, dtab.data_ptr(), out.t.data_ptr(), dpar.data_ptr(), s.hidden,
               s.q8_row_bytes, T)
    assert to_f32(out.t).tobytes() == want.tobytes()
    out.check()
    one = Guarded((s.hidden,), torch.float32)
    lib().call("matvec_q8_0_embed", st, dtab.data_ptr(), one.t.data_ptr(), int(ids[3]), s.hidden, s.q8_row_bytes)
    assert to_f32(one.t).tobytes() == want[3].tobytes()
    lib().call("matvec_q8_0_embed_p", st, dtab.data_ptr(), one.t.data_ptr(), dpar[5].data_ptr(), s.hidden,
               s.q8_row_bytes)
    assert to_f32(one.t).tobytes() == want[5].tobytes()
    one.check()


def test_embedding_vocab_guard():
    table = synth.q8_0_table("t.e3.table", 16, 64)
    ids = np.array([3, 16, 2, 4000000000], np.uint32)
    out = Guarded((4, 64), torch.float32)
    ops.embed_q8_0(to_dev(table), to_dev(ids.view(np.int32)), 64, out.t, vocab=16)
    got = to_f32(out.t)
    assert not got[1].any() and not got[3].any() and got[0].any() and got[2].any()
    out.check()


# ---- quantizers --------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(1, 32), (5, 256), (3, 2048), (4, 96)])
def test_quantizers(orc, rows, cols):
    x = synth.act("t.qz.x", rows, cols) * np.float32(10.0) ** synth.rng("t.qz.e").integers(-4, 3, size=(rows, 1))
    x = x.astype(np.float32)
    x[0, :32] = 0
    st = torch.cuda.current_stream().cuda_stream
    dx = to_dev(x)
    wq, wd = orc.quantize_i8_rows(x)
    xq, xd = Guarded((rows, cols), torch.int8), Guarded((rows, cols // 32), torch.float32)
    ops.quantize_q8_rows(dx, xq.t, xd.t)
    assert xq.t.cpu().numpy().tobytes() == wq.tobytes() and to_f32(xd.t).tobytes() == wd.tobytes()
    xq.check(), xd.check()
    q8 = Guarded((rows, cols // 32 * 34), torch.uint8)
    ops.encode_q8_0(dx, q8.t)
    assert q8.t.cpu().numpy().tobytes() == orc.encode_q8_0_rows(x).tobytes()
    q8.check()
    if cols % 64 == 0:  # K-blocked [cols / 64][T][64], scales [cols / 32][T]
        kq, kd = Guarded((cols // 64, rows, 64), torch.int8), Guarded((cols // 32, rows), torch.float32)
        lib().call("quantize_q8_kblocked", st, dx.data_ptr(), kq.t.data_ptr(), kd.t.data_ptr(), cols, rows)
        assert kq.t.cpu().numpy().tobytes() == wq.reshape(rows, cols // 64, 64).transpose(1, 0, 2).tobytes()
        assert to_f32(kd.t).tobytes() == np.ascontiguousarray(wd.T).tobytes()
        kq.check(), kd.check()
    # two int8 levels (halo_q8x_cols): second level quantizes x - q * s with the same recipe
    q1, s1 = Guarded((rows, cols), torch.int8), Guarded((rows, cols // 32), torch.float32)
    q2, s2 = Guarded((rows, cols), torch.int8), Guarded((rows, cols // 32), torch.float32)
    lib().call("q8x_cols", st, dx.data_ptr(), cols, cols, q1.t.data_ptr(), s1.t.data_ptr(), q2.t.data_ptr(),
               s2.t.data_ptr(), rows)
    assert q1.t.cpu().numpy().tobytes() == wq.tobytes()
    resid = (x.reshape(rows, -1, 32) - wq.reshape(rows, -1, 32).astype(np.float32) * wd[..., None]).reshape(rows, cols)
    rq, rd = orc.quantize_i8_rows(resid.astype(np.float32))
    assert q2.t.cpu().numpy().tobytes() == rq.tobytes() and to_f32(s2.t).tobytes() == rd.tobytes()


@pytest.mark.parametrize("B,hc,h", [(1, 4, 2048), (3, 4, 2560), (8, 2, 96), (2, 8, 36)])
def test_hc_norm_q8x(orc, B, hc, h):
    """halo_hc_norm_q8x (src/kernels/batch_decode.hip:977-999): xn = (res x scale of the stream) x norm_w, stored,
    then two int8 levels per 32 values. xn is bit-exact (two fp32 products, no contraction); codes and scales are
    bit-exact against the quantizer recipe run on xn. h = 36 leaves blocks that straddle two streams."""
    D = hc * h
    res = (synth.act("t.hq.res", B, D) * 3).astype(np.float32)
    scale = np.abs(synth.act("t.hq.sc", B, hc)).astype(np.float32) + np.float32(0.25)
    nw = (1 + 0.1 * synth.act("t.hq.w", 1, D)[0]).astype(np.float32)
    res[0, :32] = 0
    st = torch.cuda.current_stream().cuda_stream
    xn = Guarded((B, D), torch.float32)
    q1, s1 = Guarded((B, D), torch.int8), Guarded((B, D // 32), torch.float32)
    q2, s2 = Guarded((B, D), torch.int8), Guarded((B, D // 32), torch.float32)
    d_res, d_sc, d_w = to_dev(res), to_dev(scale), to_dev(nw)
    lib().call("hc_norm_q8x", st, d_res.data_ptr(), d_sc.data_ptr(), d_w.data_ptr(), xn.t.data_ptr(), hc, h,
               q1.t.data_ptr(), s1.t.data_ptr(), q2.t.data_ptr(), s2.t.data_ptr(), B)
    want = (res * np.repeat(scale, h, axis=1)) * nw[None, :]
    got = to_f32(xn.t)
    assert got.tobytes() == want.astype(np.float32).tobytes()
    wq, wd = orc.quantize_i8_rows(got)
    assert q1.t.cpu().numpy().tobytes() == wq.tobytes() and to_f32(s1.t).tobytes() == wd.tobytes()
    resid = (got.reshape(B, -1, 32) - wq.reshape(B, -1, 32).astype(np.float32) * wd[..., None]).reshape(B, D)
    rq, rd = orc.quantize_i8_rows(resid.astype(np.float32))
    assert q2.t.cpu().numpy().tobytes() == rq.tobytes() and to_f32(s2.t).tobytes() == rd.tobytes()
    for g in (xn, q1, s1, q2, s2):
        g.check()
    # the same through the scalar kernel (an unaligned xn)
    buf = torch.zeros(B * D + 1, device=DEV)
    lib().call("hc_norm_q8x", st, d_res.data_ptr(), d_sc.data_ptr(), d_w.data_ptr(), buf[1:].data_ptr(), hc, h,
               q1.t.data_ptr(), s1.t.data_ptr(), q2.t.data_ptr(), s2.t.data_ptr(), B)
    assert to_f32(buf[1:]).reshape(B, D).tobytes() == got.tobytes()
    assert q1.t.cpu().numpy().tobytes() == wq.tobytes() and q2.t.cpu().numpy().tobytes() == rq.tobytes()
    with pytest.raises(HaloError, match="does not divide|cols % 32"):
        lib().call("hc_norm_q8x", st, d_res.data_ptr(), d_sc.data_ptr(), d_w.data_ptr(), xn.t.data_ptr(), 3, 10,
                   q1.t.data_ptr(), s1.t.data_ptr(), q2.t.data_ptr(), s2.t.data_ptr(), 1)


@pytest.mark.parametrize("ddt", ["f32", "f16"])
def test_copy_at_entries(ddt):
    """halo_copy_at_y (src/kernels/batch_decode.hip:1700-1707): every session appends its row to its own cache,
    found through a table of device addresses, at the position in its own step parameters."""
    B, n, rows, pstride, slot, tstride, tslot = 3, 520, 6, 16, 1, 4, 2
    tdt = torch.float32 if ddt == "f32" else torch.float16
    src_stride = n + 8
    src = synth.act("t.cay.src", B, src_stride)
    caches = [torch.full((rows, n), -1.0, device=DEV, dtype=tdt) for _ in range(B)]
    pos = [4, 0, 5]
    params = np.zeros((B, pstride), np.uint32)
    params[:, slot] = pos
    tab = np.zeros((B, tstride), np.uint64)
    for e in range(B):
        tab[e, tslot] = caches[e].data_ptr()
    d_tab, d_par, d_src = torch.from_numpy(tab.view(np.int64)).to(DEV), to_dev(params.view(np.int32)), to_dev(src)
    st = torch.cuda.current_stream().cuda_stream
    lib().call("copy_at_y", st, d_tab.data_ptr(), tstride, tslot, 0 if ddt == "f32" else 1, d_src.data_ptr(),
               d_par.data_ptr(), slot, n, n, src_stride, pstride, B)
    for e in range(B):
        got = caches[e].float().cpu().numpy()
        want = np.full((rows, n), -1.0, np.float32)
        want[pos[e]] = src[e, :n] if ddt == "f32" else src[e, :n].astype(np.float16).astype(np.float32)
        assert got.tobytes() == want.tobytes(), f"entry {e}"
    if ddt == "f32":  # by name, as the batched decoder launches it: grid (ceil(n / 256), B)
        from halo_flash_b200.device import Arg, Device
        dev = Device.create(0)
        for c in caches:
            c.fill_(-1.0)
        torch.cuda.synchronize()  # the device object launches on its own stream
        b_tab, b_src, b_par = dev.alloc(tab.nbytes), dev.alloc(src.nbytes), dev.alloc(params.nbytes)
        dev.upload(b_tab, 0, tab), dev.upload(b_src, 0, src), dev.upload(b_par, 0, params)
        dev.launch(dev.kernel("halo_copy_at_y"), ((n + 255) // 256, B), (256,),
                   [Arg.Buf(b_tab), Arg.U32(tstride), Arg.U32(tslot), Arg.Buf(b_src), Arg.Buf(b_par), Arg.U32(slot),
                    Arg.U32(n), Arg.U32(n), Arg.U32(src_stride), Arg.U32(pstride)])
        dev.synchronize()
        for e in range(B):
            assert caches[e][pos[e]].cpu().numpy().tobytes() == src[e, :n].tobytes()


# ---- empty and ragged inputs ---------------------------------------------------------------
def test_empty_inputs_are_no_ops():
    e = torch.empty(0, 256, device=DEV)
    w = torch.ones(256, device=DEV)
    ops.rmsnorm(e, w, 1e-6)
    ops.l2norm(e, 1e-6)
    ops.silu_mul(e, e.clone())
    ops.gated_norm(e, w, e.clone(), 1e-6)
    ops.rope(torch.empty(0, 4, 64, device=DEV), None, 16, 1e7)
    ops.embed_q8_0(torch.zeros(4, 272, dtype=torch.uint8, device=DEV), torch.zeros(0, dtype=torch.int32, device=DEV),
                   256, torch.empty(0, 256, device=DEV))
    torch.cuda.synchronize()


# ---- full-size inputs: sampled rows against the oracle plus size-independent properties ------
def test_full_size_prefill_properties(orc):
    s, T = synth.FULL, 4096
    g = torch.Generator(device=DEV).manual_seed(synth.SEED)
    pick = np.unique(synth.rng("t.fs.pick").integers(0, T, size=48))
    # add + RMSNorm, bf16, with the Q8_0 epilogue
    res = torch.randn(T, s.hidden, device=DEV, generator=g).bfloat16()
    delta = torch.randn(T, s.hidden, device=DEV, generator=g).bfloat16()
    w = to_dev(synth.norm_w("t.fs.w", s.hidden))
    res0 = res.clone()
    xn = torch.empty_like(res)
    q8 = torch.empty(T, s.q8_row_bytes, dtype=torch.uint8, device=DEV)
    ops.add_rmsnorm(res, delta, w, s.eps, xn=xn, q8_0=q8)
    stored = oracle.round_bf16(to_f32(res0[pick]) + to_f32(delta[pick]))
    assert np.array_equal(bits16(res[pick]), oracle.bf16_bits(stored))
    want = orc.rmsnorm_rows(stored.copy(), ONE + to_f32(w), s.eps)
    assert_bf16_within_1ulp(bits16(xn[pick]), want, "full-size xn")
    # property: mean square of xn / (1 + w) is 1 for every row (up to bf16 rounding)
    ms = ((xn.float() / (1 + w)) ** 2).mean(dim=1)
    assert float((ms - 1).abs().max()) < 2e-2
    # property: Q8_0 decode of the epilogue reproduces xn within half a quantization step
    deq = torch.empty(T, s.hidden, device=DEV)
    ops.embed_q8_0(q8, torch.arange(T, dtype=torch.int32, device=DEV), s.hidden, deq)
    amax = xn.float().view(T, -1, 32).abs().amax(dim=2, keepdim=True)
    assert bool(((deq.view(T, -1, 32) - xn.float().view(T, -1, 32)).abs() <= amax / 127 * 0.5 * 1.02 + amax * 2 ** -8).all())
    # gated norm at the DeltaNet output shape, bf16
    o = torch.randn(T * s.v_heads, s.lin_dim, device=DEV, generator=g).bfloat16()
    z = torch.randn(T * s.v_heads, s.lin_dim, device=DEV, generator=g).bfloat16()
    gw = to_dev(synth.gated_w("t.fs.gw", s.lin_dim))
    y = torch.empty_like(o)
    ops.gated_norm(o, gw, z, s.eps, y=y)
    rows = np.unique(synth.rng("t.fs.rows").integers(0, T * s.v_heads, size=256))
    wantg = orc.gated_norm_rows(to_f32(o[rows]), to_f32(gw), to_f32(z[rows]), s.eps, 0)
    assert_bf16_within_1ulp(bits16(y[rows]), wantg, "full-size gated norm")
    # L2 norm: unit rows, and idempotent up to rounding
    qk = torch.randn(T * 2 * s.k_heads, s.lin_dim, device=DEV, generator=g)
    ops.l2norm(qk, s.eps)
    assert float(((qk * qk).sum(dim=1) - 1).abs().max()) < 1e-4
    again = qk.clone()
    ops.l2norm(again, s.eps)
    assert float((again - qk).abs().max()) < 1e-5
    # RoPE: rotation preserves each pair's norm and leaves dims beyond rot untouched
    q = torch.randn(T, s.q_heads, s.head_dim, device=DEV, generator=g)
    q0 = q.clone()
    ops.rope(q, None, s.rot, s.theta, pos0=262144 - T)
    h = s.rot // 2
    n0 = q0[..., :h] ** 2 + q0[..., h:s.rot] ** 2
    n1 = q[..., :h] ** 2 + q[..., h:s.rot] ** 2
    assert float(((n1 - n0).abs() / (n0 + 1e-12)).max()) < 1e-5
    assert torch.equal(q[..., s.rot:], q0[..., s.rot:])
    sel = pick[:8]
    wantq = orc.rope_rows(to_f32(q0[sel]), (262144 - T + sel).astype(np.uint32), s.rot, s.theta)
    check_rope(to_f32(q[sel]), wantq, to_f32(q0[sel]), s.rot, "full-size rope")
    # routed SwiGLU rows [T * top_k, ff], bf16: linear in `up`
    gate = torch.randn(T * s.top_k, s.ff, device=DEV, generator=g).bfloat16()
    up = torch.randn(T * s.top_k, s.ff, device=DEV, generator=g).bfloat16()
    hout = torch.empty_like(gate)
    ops.silu_mul(gate, up, y=hout)
    prow = np.unique(synth.rng("t.fs.pairs").integers(0, T * s.top_k, size=256))  # (token, slot) pair rows
    wanth = orc.silu_mul(to_f32(gate[prow]), to_f32(up[prow]))
    assert_bf16_within_1ulp(bits16(hout[prow]), wanth, "full-size swiglu")
    h2 = torch.empty(T * s.top_k, s.ff, device=DEV)
    ops.silu_mul(gate, (up.float() * 2).bfloat16(), y=h2)
    h1 = torch.empty(T * s.top_k, s.ff, device=DEV)
    ops.silu_mul(gate, up, y=h1)
    assert torch.equal(h2, 2 * h1), "SiLU(g) * up is exactly linear under doubling of up"
    # embedding: equal ids give equal rows; rows equal the oracle's
    table = to_dev(synth.q8_0_table("t.fs.table", 2048, s.hidden))
    ids = torch.randint(0, 2048, (T,), device=DEV, generator=g, dtype=torch.int32)
    ids[1] = ids[0]
    emb = torch.empty(T, s.hidden, device=DEV, dtype=torch.bfloat16)
    ops.embed_q8_0(table, ids, s.hidden, emb)
    assert torch.equal(emb[0], emb[1])
    wante = orc.embed_q8_0_rows(table.cpu().numpy(), ids[pick].cpu().numpy().view(np.uint32), s.hidden)
    assert np.array_equal(bits16(emb[pick]), oracle.bf16_bits(wante))


@pytest.mark.parametrize("rows", [64, 1778, 28416, 28418])
def test_lean_and_general_norm_kernels_agree_bit_for_bit(rows):
    """The lean kernel (dense, full grid) and the general kernel compute the same bits. The row counts sit on the
    lean kernels' launch-shape boundaries: 64 rows fit one wave of resident CTAs, 1778 rows of 2048 are one CTA more
    than a wave (the first CTA then hints its successor's rows to L2), 28 416 rows are exactly sixteen waves (the
    longest launch that still does so) and 28 418 one CTA more."""
    s = synth.FULL
    res, delta = to_dev(synth.act("t.lg.res", rows, s.hidden), "bf16"), to_dev(synth.act("t.lg.delta", rows, s.hidden), "bf16")
    w = to_dev(synth.norm_w("t.lg.w", s.hidden))
    outs = []
    for force in (0, 1):
        lib().tune("norm_force_general", force)
        try:
            r = res.clone()
            xn = torch.empty_like(r)
            q8 = torch.empty(rows, s.q8_row_bytes, dtype=torch.uint8, device=DEV)
            ops.add_rmsnorm(r, delta, w, s.eps, xn=xn, q8_0=q8)
            heads = 32 if rows <= 2048 else 2  # the one-head rows: 2048 of them and more already span several waves
            qk = to_dev(synth.act("t.lg.qk", rows * heads, s.lin_dim), "bf16")
            ops.l2norm(qk, s.eps)
            o = to_dev(synth.act("t.lg.o", rows * heads, s.lin_dim), "bf16")
            z = to_dev(synth.act("t.lg.z", rows * heads, s.lin_dim), "bf16")
            ops.gated_norm(o, to_dev(synth.gated_w("t.lg.gw", s.lin_dim)), z, s.eps)
            r2, xn2 = res.clone(), torch.empty_like(res)
            ops.add_rmsnorm(r2, delta, w, s.eps, xn=xn2)  # the kernel without an epilogue
            outs.append((r, xn, q8, qk, o, r2, xn2))
        finally:
            lib().tune("norm_force_general", 0)
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_q_and_k_norm_rope_in_one_launch(orc):
    """halo_b200_norm_rope_qk_ex == the two single-tensor launches bit for bit, and matches the oracle;
    also the q|gate split with K appended to a cache."""
    s, T, pos0 = synth.FULL, 21, 4000
    hd = s.head_dim
    q = rounded(synth.act("t.qk.q", T, s.q_heads, hd), "bf16")
    k = rounded(synth.act("t.qk.k", T, s.kv_heads, hd), "bf16")
    wq, wk = synth.norm_w("t.qk.wq", hd), synth.norm_w("t.qk.wk", hd)
    dwq, dwk = to_dev(wq), to_dev(wk)
    q1, k1 = to_dev(q, "bf16"), to_dev(k, "bf16")
    ops.norm_rope(q1.view(-1, hd), dwq, s.eps, s.rot, s.theta, s.q_heads, pos0=pos0)
    ops.norm_rope(k1.view(-1, hd), dwk, s.eps, s.rot, s.theta, s.kv_heads, pos0=pos0)
    q2, k2 = to_dev(q, "bf16"), to_dev(k, "bf16")
    used = Guarded((T,), torch.int32)
    ops.norm_rope_qk(q2, k2, dwq, dwk, s.eps, s.rot, s.theta, pos0=pos0, pos_out=used.t)
    assert torch.equal(q1, q2) and torch.equal(k1, k2)
    assert np.array_equal(used.t.cpu().numpy(), np.arange(pos0, pos0 + T))
    used.check()
    pos = np.arange(pos0, pos0 + T, dtype=np.uint32)
    wantq = orc.rope_rows(orc.rmsnorm_rows(q.reshape(-1, hd).copy(), ONE + wq, s.eps).reshape(q.shape), pos, s.rot, s.theta)
    wantk = orc.rope_rows(orc.rmsnorm_rows(k.reshape(-1, hd).copy(), ONE + wk, s.eps).reshape(k.shape), pos, s.rot, s.theta)
    assert_bf16_rope(bits16(q2), wantq, "q")
    assert_bf16_rope(bits16(k2), wantk, "k")
    # fp32, interleaved q|gate rows, K cache append, tiny shapes (4 Q / 2 KV heads x 64, rot 16)
    c, T2 = synth.C1, 9
    qg = synth.act("t.qk.qg", T2 * c.q_heads, 2 * c.head_dim)
    kk = synth.act("t.qk.kk", T2, c.kv_heads, c.head_dim)
    w1, w2 = synth.norm_w("t.qk.w1", c.head_dim), synth.norm_w("t.qk.w2", c.head_dim)
    qo, gate = Guarded((T2, c.q_heads, c.head_dim), torch.float32), Guarded((T2 * c.q_heads, c.head_dim), torch.float32)
    cache = Guarded((T2, c.kv_heads, c.head_dim), torch.float32)
    dk = to_dev(kk)
    ops.norm_rope_qk(to_dev(qg), dk, to_dev(w1), to_dev(w2), c.eps, c.rot, c.theta, q_out=qo.t, q_gate=gate.t,
                     k_cache=cache.t, q_row_stride=2 * c.head_dim, pos0=77)
    p2 = np.arange(77, 77 + T2, dtype=np.uint32)
    wq2 = orc.rope_rows(orc.rmsnorm_rows(np.ascontiguousarray(qg[:, :c.head_dim]), ONE + w1, c.eps).reshape(T2, c.q_heads, -1), p2, c.rot, c.theta)
    wk2 = orc.rope_rows(orc.rmsnorm_rows(kk.reshape(-1, c.head_dim).copy(), ONE + w2, c.eps).reshape(kk.shape), p2, c.rot, c.theta)
    assert_rows_close(to_f32(qo.t).reshape(-1, c.head_dim), wq2.reshape(-1, c.head_dim), what="q of q|gate")
    assert_rows_close(to_f32(dk).reshape(-1, c.head_dim), wk2.reshape(-1, c.head_dim), what="k")
    assert to_f32(gate.t).tobytes() == np.ascontiguousarray(qg[:, c.head_dim:]).tobytes()
    assert torch.equal(cache.t, dk)
    for gd in (qo, gate, cache):
        gd.check()


def test_swiglu_several_tensors_in_one_launch(orc):
    shapes = [(4096 * 3, ), (7, 512), (1, 8), (33, 5)]  # the last two exercise the tile tail and the scalar tail
    gs = [rounded(synth.act(f"t.mm.g{i}", *sh) * 3, "bf16") for i, sh in enumerate(shapes)]
    us = [rounded(synth.act(f"t.mm.u{i}", *sh), "bf16") for i, sh in enumerate(shapes)]
    outs = [Guarded(sh, torch.bfloat16) for sh in shapes]
    ops.silu_mul_multi([(to_dev(g, "bf16"), to_dev(u, "bf16")) for g, u in zip(gs, us)], [o.t for o in outs])
    for g, u, o in zip(gs, us, outs):
        want = orc.silu_mul(g.copy().reshape(-1), u.reshape(-1))
        assert_bf16_within_1ulp(bits16(o.t).reshape(-1), want, "multi swiglu")
        o.check()
    single = Guarded(shapes[0], torch.bfloat16)
    ops.silu_mul(to_dev(gs[0], "bf16"), to_dev(us[0], "bf16"), y=single.t)
    assert torch.equal(single.t, outs[0].t)


def test_rotation_table_path_equals_in_kernel_sincos(orc):
    """norm_rope_qk_table_ex (cos / sin read from a precomputed table) == norm_rope_qk_ex bit for bit;
    the table itself holds cos / sin of float(pos) * inv_freq within 1e-6 of the CPU's libm."""
    s, T, pos0 = synth.FULL, 37, 262144 - 37
    q = rounded(synth.act("t.tb.q", T, s.q_heads, s.head_dim), "bf16")
    k = rounded(synth.act("t.tb.k", T, s.kv_heads, s.head_dim), "bf16")
    wq, wk = to_dev(synth.norm_w("t.tb.wq", s.head_dim)), to_dev(synth.norm_w("t.tb.wk", s.head_dim))
    table = Guarded((T, 2, s.rot // 2), torch.float32)
    used = torch.zeros(T, dtype=torch.int32, device=DEV)
    ops.rope_table(table.t, s.rot, s.theta, pos0=pos0, pos_out=used)
    table.check()
    assert np.array_equal(used.cpu().numpy(), np.arange(pos0, pos0 + T))
    inv = orc.rope_inv_freq(s.rot, s.theta)
    ang = (np.arange(pos0, pos0 + T, dtype=np.uint32).astype(np.float32)[:, None] * inv[None, :]).astype(np.float32)
    got = to_f32(table.t)
    assert np.abs(got[:, 0] - np.cos(ang.astype(np.float64))).max() < 1e-6
    assert np.abs(got[:, 1] - np.sin(ang.astype(np.float64))).max() < 1e-6
    q1, k1 = to_dev(q, "bf16"), to_dev(k, "bf16")
    ops.norm_rope_qk(q1, k1, wq, wk, s.eps, s.rot, s.theta, pos0=pos0)
    q2, k2 = to_dev(q, "bf16"), to_dev(k, "bf16")
    ops.norm_rope_qk_table(q2, k2, wq, wk, s.eps, s.rot, table.t)
    assert torch.equal(q1, q2) and torch.equal(k1, k2)
    q3 = to_dev(q, "bf16")
    ops.norm_rope_qk_table(q3, None, wq, None, s.eps, s.rot, table.t)
    assert torch.equal(q1, q3)
    # T = 32 fills the lean kernel's grid exactly; its result equals the general kernel's
    T2 = 32
    qa = rounded(synth.act("t.tb.qa", T2, s.q_heads, s.head_dim), "bf16")
    ka = rounded(synth.act("t.tb.ka", T2, s.kv_heads, s.head_dim), "bf16")
    tab2 = ops.rope_table(torch.empty(T2, 2, s.rot // 2, device=DEV), s.rot, s.theta, pos0=100000)
    res = []
    for force in (0, 1):
        lib().tune("norm_force_general", force)
        try:
            qd, kd = to_dev(qa, "bf16"), to_dev(ka, "bf16")
            ops.norm_rope_qk_table(qd, kd, wq, wk, s.eps, s.rot, tab2)
            res.append((qd, kd))
        finally:
            lib().tune("norm_force_general", 0)
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])
    pos = np.arange(100000, 100000 + T2, dtype=np.uint32)
    wantq = orc.rope_rows(orc.rmsnorm_rows(qa.reshape(-1, s.head_dim).copy(), ONE + to_f32(wq), s.eps).reshape(qa.shape),
                          pos, s.rot, s.theta)
    assert_bf16_rope(bits16(res[0][0]), wantq, "lean norm+rope q")


def test_dependent_launch_orders_the_chain():
    """The kernels are launched so that each may be scheduled while its predecessor drains and
    order themselves on the device. The 230-launch chain, whose residual stream is read and
    rewritten by every second launch, must give the same bits with that overlap (eager and as a
    replayed graph) as with plain stream-ordered launches."""
    from halo_flash_b200.chain import LayerChain

    def run(pdl, graph):
        lib().tune("pdl", pdl)
        try:
            ch = LayerChain(synth.FULL, 512, pos0=1000, vocab=4096)
            if graph:
                ch.capture()
                ch.replay()
                ch.replay()
            else:
                ch.step()
            torch.cuda.synchronize()
            outs = [ch.res, ch.xn, ch.h_s, ch.h_r] + [t for bo in ch.sets for t in (bo.qk, bo.y, bo.q, bo.k)]
            return [t.clone() for t in outs]
        finally:
            lib().tune("pdl", 1)

    # q/k/qk are normalized in place, so a chain object is used for exactly one step (or one
    # capture + two replays, compared against the same sequence without overlap)
    plain, overlapped = run(0, False), run(1, False)
    for a, b in zip(plain, overlapped):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    plain_g, overlapped_g = run(0, True), run(1, True)
    for a, b in zip(plain_g, overlapped_g):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_decode_batch_with_device_step_params(orc):
    """Config 2: B = 8 decode tokens, the full-size 151 936-row Q8_0 table, token ids and positions up to
    262 143 read from device memory (rows 16 uint32 apart), one captured chain step replayed after the
    parameters change. The gather is bit-exact, the rotation matches the oracle at each entry's position."""
    from halo_flash_b200.chain import LayerChain
    s, B = synth.FULL, 8
    ch = LayerChain(s, B, pos0=0, step_params=True, q8_epilogue=True)
    ch.capture()
    rng = synth.rng("t.decode")
    table = ch.table.cpu().numpy()
    for _ in range(3):
        ids = rng.integers(0, s.vocab, size=B).astype(np.int32)
        ids[0], ids[1] = 0, s.vocab - 1
        pos = rng.integers(0, s.max_pos, size=B).astype(np.int32)
        pos[0], pos[1] = s.max_pos - 1, 0
        p = np.zeros((B, 16), np.int32)
        p[:, 0], p[:, 1] = ids, pos
        q0 = ch.sets[3 % len(ch.sets)].q.clone()  # layer 3 is the first GQA layer
        ch.params.copy_(torch.from_numpy(p).to(DEV))
        # the embedding gather alone, then one rotation through the step's table
        ops.embed_q8_0(ch.table, ch.params, s.hidden, ch.res, id_stride=16, id_slot=0, vocab=s.vocab)
        want = orc.embed_q8_0_rows(table, ids.view(np.uint32), s.hidden)
        assert np.array_equal(bits16(ch.res), oracle.bf16_bits(want))
        ops.rope_table(ch.rope_tab, s.rot, s.theta, params=ch.params, pstride=16, slot=1)
        q = q0.float()
        w_q = torch.zeros(s.head_dim, device=DEV)
        qn = q.clone()
        ops.norm_rope_qk_table(qn, None, w_q, w_q, s.eps, s.rot, ch.rope_tab, one_plus=True)
        wantq = orc.rmsnorm_rows(to_f32(q).reshape(-1, s.head_dim).copy(), np.ones(s.head_dim, np.float32), s.eps)
        wantq = orc.rope_rows(wantq.reshape(B, s.q_heads, s.head_dim), pos.view(np.uint32), s.rot, s.theta)
        assert_rows_close(to_f32(qn).reshape(-1, s.head_dim), wantq.reshape(-1, s.head_dim), what="decode rope at device positions")
        # the captured step at these parameters equals the eager step
        sets0 = [[t.clone() for t in bo.inputs()] for bo in ch.sets]
        ch.replay()
        torch.cuda.synchronize()
        got = (ch.res.clone(), ch.xn_q8.clone(), ch.h_r.clone())
        # the Q8_0 epilogue of the last add + norm: blocks bit-exact against the oracle encoder run on the
        # oracle's norm of the residual the GPU stored (codes may differ only where xn differs; so decode both)
        stored = to_f32(ch.res)
        want_xn = orc.rmsnorm_rows(stored.copy(), ONE + to_f32(ch.w_post[-1]), s.eps)
        deq = torch.empty(B, s.hidden, device=DEV)
        ops.embed_q8_0(ch.xn_q8, torch.arange(B, dtype=torch.int32, device=DEV), s.hidden, deq)
        amax = np.abs(want_xn).reshape(B, -1, 32).max(axis=2, keepdims=True)
        assert np.all(np.abs(to_f32(deq).reshape(B, -1, 32) - want_xn.reshape(B, -1, 32)) <= amax / 127 * 0.51 + amax * 1e-3)
        for bo, saved in zip(ch.sets, sets0):  # q / k / qk were normalized in place: restore, then run eagerly
            for t, v in zip(bo.inputs(), saved):
                t.copy_(v)
        ch.step()
        torch.cuda.synchronize()
        for a, b in zip(got, (ch.res, ch.xn_q8, ch.h_r)):
            assert torch.equal(a, b)
        for bo, saved in zip(ch.sets, sets0):
            for t, v in zip(bo.inputs(), saved):
                t.copy_(v)


def test_no_staging_wait_ran_out():
    """Every wait of the persistent, shared-memory-staging kernels (conv + SiLU + L2 norm, fused norm + RoPE) is
    bounded; one that runs out is counted. After the tests collected before this one: zero."""
    import ctypes as C
    n = C.c_uint(123)
    err = C.create_string_buffer(256)
    f = lib().cdll.halo_b200_stage_timeouts
    f.restype, f.argtypes = C.c_int, [C.POINTER(C.c_uint), C.c_char_p, C.c_size_t]
    assert f(C.byref(n), err, len(err)) == 0, err.value
    assert n.value == 0
