"""Every reference kernel name the library replaces, launched BY NAME the way the reference's engine
launches it (rt::Device::Kernel + Launch: the kernel's own ordered argument list, its grid and block;
src/engine/qwen35_gpu.cpp:163-251, src/engine/prefill_chunk.cpp:380-713, src/engine/batch_decode.cpp:429-438)
and compared with the CPU oracle at the tolerance of its op.

The table below has one case per name; `test_every_kernel_name_has_a_case` (no GPU needed) fails when
`halo_b200_kernel_name()` lists a name without one. The wrapper is where argument order, dtype mapping
and grid decoding can go wrong, so each case goes through `halo_b200_launch`, not a typed entry point.
Cross-checks the reference itself makes between kernel forms (tests/gpu/quant_gpu_test.cpp:2361-2422,
2752-2814) are repeated: the fp16-emitting norms give the plain norm's fp32 output bit for bit and its
fp16 rounding; the one-warp-per-row gated norm (h128w) equals the block form bit for bit.
"""
import numpy as np
import pytest

import oracle
from conftest import assert_bf16_within_1ulp, assert_rows_close
from halo_flash_b200 import lib, synth
from halo_flash_b200.device import Arg, Device

EPS = 1e-6
CASES = {}


def case(*names):
    def deco(fn):
        for n in names:
            assert n not in CASES, n
            CASES[n] = fn
        return fn
    return deco


class Box:
    """A device plus the upload / download / launch shorthands the cases use."""

    def __init__(self, dev, orc):
        self.dev, self.orc = dev, orc

    def up(self, a):
        a = np.ascontiguousarray(a)
        b = self.dev.alloc(a.nbytes)
        self.dev.upload(b, 0, a)
        return b

    def new(self, nbytes, fill=None):
        b = self.dev.alloc(nbytes)
        if fill is not None:
            self.dev.fill(b, fill)
        return b

    def dl(self, b, shape, dtype=np.float32):
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        return self.dev.download(b, 0, n, dtype).reshape(shape)

    def run(self, name, grid, block, args):
        self.dev.launch(self.dev.kernel(name), grid, block, args)


B_, U, F, U64 = Arg.Buf, Arg.U32, Arg.F32, Arg.U64


def f16r(a):
    return a.astype(np.float16).astype(np.float32)


def as16(a, dt):
    """fp32 array -> (bits to upload, the fp32 values those bits hold) for dt in f32 / f16 / bf16."""
    if dt == "f16":
        return a.astype(np.float16), f16r(a)
    if dt == "bf16":
        return oracle.bf16_bits(a), oracle.round_bf16(a)
    return a.astype(np.float32), a.astype(np.float32)


def from16(bits, dt):
    return bits.astype(np.float32) if dt == "f16" else oracle.bf16_to_f32(bits) if dt == "bf16" else bits


def ulp16(got_bits, want_f32, dt):
    """Distance, in units of the 16-bit type, between stored bits and the rounding of want."""
    if dt == "bf16":
        a, b = got_bits.astype(np.int32), oracle.bf16_bits(want_f32).astype(np.int32)
    else:
        a, b = got_bits.view(np.uint16).astype(np.int32), want_f32.astype(np.float16).view(np.uint16).astype(np.int32)
    order = lambda v: np.where(v & 0x8000, 0x8000 - (v & 0x7FFF) - 1, 0x8000 + v)
    return np.abs(order(a) - order(b))


def sigmoid_ref(orc, x):
    return np.array([orc._call("orc_sigmoid", float(v)) for v in np.asarray(x, np.float32).reshape(-1)],
                    np.float32).reshape(np.shape(x))


def silu_ref(orc, x):
    return np.array([orc._call("orc_silu", float(v)) for v in np.asarray(x, np.float32).reshape(-1)],
                    np.float32).reshape(np.shape(x))


def close_elt(got, want, rel=1e-5, what=""):
    assert np.all(np.abs(got.astype(np.float64) - want) <= rel * np.abs(want) + 1e-30), what


SUFFIX = {"": "f32", "_r16": "f16", "_rb": "bf16"}


# ---- group 1 ---------------------------------------------------------------------------------
@case("halo_add", "halo_axpy")
def _add(b, name):
    n = 1000
    y, x = synth.act("n.add.y", n), synth.act("n.add.x", n)
    by, bx = b.up(y), b.up(x)
    if name == "halo_add":
        b.run(name, ((n + 255) // 256,), (256,), [B_(by), B_(bx), U(n)])
        assert b.dl(by, (n,)).tobytes() == (y + x).tobytes()
    else:
        a = np.float32(0.37)
        b.run(name, ((n + 255) // 256,), (256,), [B_(by), B_(bx), F(float(a)), U(n)])
        assert b.dl(by, (n,)).tobytes() == (y + a * x).astype(np.float32).tobytes(), "y + a x: product and sum round separately"


@case("halo_rmsnorm")
def _rmsnorm(b, name):
    rows, d = 3, 2048
    x, w = synth.act("n.rms.x", rows, d), (1 + synth.norm_w("n.rms.w", rows * d)).reshape(rows, d)
    bx, bw, by = b.up(x), b.up(w), b.new(x.nbytes)
    b.run(name, (rows,), (256,), [B_(bx), B_(bw), B_(by), U(d), F(EPS), U(d)])  # vector r uses gamma row r
    want = np.stack([b.orc.rmsnorm_rows(x[r:r + 1].copy(), w[r], EPS)[0] for r in range(rows)])
    assert_rows_close(b.dl(by, (rows, d)), want, what=name)
    b.run(name, (rows,), (256,), [B_(bx), B_(bw), B_(bx), U(d), F(EPS), U(0)])  # shared gamma, in place
    assert_rows_close(b.dl(bx, (rows, d)), b.orc.rmsnorm_rows(x.copy(), w[0], EPS), what=name + " in place")


@case("halo_rmsnorm_rows", "halo_rmsnorm_rows_r16", "halo_rmsnorm_rows_rb")
def _rmsnorm_rows(b, name):
    dt = SUFFIX[name[len("halo_rmsnorm_rows"):]]
    T, hc, d = 5, 4, 320
    bits, x = as16(synth.act("n.rr.x", T * hc, d) * 3, dt)
    w = (1 + synth.norm_w("n.rr.w", hc * d)).reshape(hc, d)
    bx, bw, by = b.up(bits), b.up(w), b.new(T * hc * d * 4)
    b.run(name, (T * hc,), (256,), [B_(bx), B_(bw), B_(by), U(d), F(EPS), U(d), U(hc)])
    want = b.orc.rmsnorm_rows(x.copy(), w, EPS, w_stride=d, w_period=hc)
    assert_rows_close(b.dl(by, (T * hc, d)), want, what=name)


@case("halo_rmsnorm_rows_h", "halo_rmsnorm_rows_h_r16", "halo_rmsnorm_rows_h_rb")
def _rmsnorm_rows_h(b, name):
    sfx = name[len("halo_rmsnorm_rows_h"):]
    dt = SUFFIX[sfx]
    T, hc, d = 6, 4, 256
    bits, x = as16(synth.act("n.rh.x", T * hc, d) * 2, dt)
    w = (1 + synth.norm_w("n.rh.w", hc * d)).reshape(hc, d)
    bx, bw = b.up(bits), b.up(w)
    # the plain form of the same dtype: its fp32 output is the yardstick (bit for bit)
    by0 = b.new(T * hc * d * 4)
    b.run("halo_rmsnorm_rows" + sfx, (T * hc,), (256,), [B_(bx), B_(bw), B_(by0), U(d), F(EPS), U(d), U(hc)])
    y0 = b.dl(by0, (T * hc, d))
    assert_rows_close(y0, b.orc.rmsnorm_rows(x.copy(), w, EPS, w_stride=d, w_period=hc), what=name + " yardstick")
    for y16_tokens in (0, T):
        by, by16 = b.new(T * hc * d * 4, 0), b.new(T * hc * d * 2, 0)
        b.run(name, (T * hc,), (256,), [B_(bx), B_(bw), B_(by), B_(by16), U(d), F(EPS), U(d), U(hc), Arg.Null, Arg.Null,
                                        U(0), U(y16_tokens)])
        assert b.dl(by, (T * hc, d)).tobytes() == y0.tobytes(), name + ": fp32 output differs from the plain form"
        h = b.dl(by16, (T * hc * d,), np.float16)
        if y16_tokens:  # K-blocked [hc d / 64][T][64]
            h = h.reshape(hc * d // 64, T, 64).transpose(1, 0, 2).reshape(T * hc, d)
        assert np.array_equal(h.reshape(T * hc, d), y0.astype(np.float16)), name + ": fp16 copy"


@case("halo_rmsnorm_y")
def _rmsnorm_y(b, name):
    batch, nvec, d, stride = 3, 4, 256, 4 * 256 + 64
    arena = synth.act("n.ry.x", batch * stride)
    w = 1 + synth.norm_w("n.ry.w", d)
    bx, bw = b.up(arena), b.up(w)
    b.run(name, (nvec, batch), (256,), [B_(bx), B_(bw), U(d), F(EPS), U(0), U(stride)])
    got = b.dl(bx, (batch, stride))
    src = arena.reshape(batch, stride)
    for e in range(batch):
        want = b.orc.rmsnorm_rows(src[e, :nvec * d].reshape(nvec, d).copy(), w, EPS)
        assert_rows_close(got[e, :nvec * d].reshape(nvec, d), want, what=f"{name} entry {e}")
        assert got[e, nvec * d:].tobytes() == src[e, nvec * d:].tobytes(), "wrote between the entries"


@case("halo_quantize_q8_rows", "halo_quantize_q8_kblocked", "halo_q8x_cols")
def _quantize(b, name):
    rows, cols = 5, 256
    x = (synth.act("n.q.x", rows, cols) * np.float32(10.0) ** synth.rng("n.q.e").integers(-3, 3, size=(rows, 1))).astype(np.float32)
    x[0, :32] = 0
    wq, wd = b.orc.quantize_i8_rows(x)
    bx = b.up(x)
    if name == "halo_quantize_q8_rows":
        bq, bd = b.new(rows * cols), b.new(rows * cols // 32 * 4)
        b.run(name, (rows,), (256,), [B_(bx), B_(bq), B_(bd), U(cols)])
        assert b.dl(bq, (rows, cols), np.int8).tobytes() == wq.tobytes() and b.dl(bd, (rows, cols // 32)).tobytes() == wd.tobytes()
    elif name == "halo_quantize_q8_kblocked":
        bq, bd = b.new(rows * cols), b.new(rows * cols // 32 * 4)
        b.run(name, (rows,), (256,), [B_(bx), B_(bq), B_(bd), U(cols), U(rows)])
        assert b.dl(bq, (cols // 64, rows, 64), np.int8).tobytes() == wq.reshape(rows, cols // 64, 64).transpose(1, 0, 2).tobytes()
        assert b.dl(bd, (cols // 32, rows)).tobytes() == np.ascontiguousarray(wd.T).tobytes()
    else:  # two int8 levels: the second quantizes x - q * s with the same recipe
        bq, bs, bq2, bs2 = b.new(rows * cols), b.new(rows * cols // 32 * 4), b.new(rows * cols), b.new(rows * cols // 32 * 4)
        b.run(name, (cols // 32, rows), (32,), [B_(bx), U(cols), U(cols), B_(bq), B_(bs), B_(bq2), B_(bs2)])
        assert b.dl(bq, (rows, cols), np.int8).tobytes() == wq.tobytes() and b.dl(bs, (rows, cols // 32)).tobytes() == wd.tobytes()
        resid = (x.reshape(rows, -1, 32) - wq.reshape(rows, -1, 32).astype(np.float32) * wd[..., None]).reshape(rows, cols)
        rq, rd = b.orc.quantize_i8_rows(resid.astype(np.float32))
        assert b.dl(bq2, (rows, cols), np.int8).tobytes() == rq.tobytes() and b.dl(bs2, (rows, cols // 32)).tobytes() == rd.tobytes()


@case("halo_hc_norm_q8x")
def _hc_norm_q8x(b, name):
    B, hc, h = 3, 4, 256
    D = hc * h
    res = (synth.act("n.hq.res", B, D) * 3).astype(np.float32)
    scale = np.abs(synth.act("n.hq.sc", B, hc)).astype(np.float32) + np.float32(0.25)
    nw = (1 + 0.1 * synth.act("n.hq.w", D)).astype(np.float32)
    bxn, bq, bs = b.new(B * D * 4), b.new(B * D), b.new(B * D // 32 * 4)
    b.run(name, (D // 32, B), (32,), [B_(b.up(res)), B_(b.up(scale)), B_(b.up(nw)), B_(bxn), U(hc), U(h), B_(bq), B_(bs),
                                      Arg.Null, Arg.Null])
    xn = b.dl(bxn, (B, D))
    assert xn.tobytes() == ((res * np.repeat(scale, h, axis=1)) * nw[None, :]).astype(np.float32).tobytes()
    wq, wd = b.orc.quantize_i8_rows(xn)
    assert b.dl(bq, (B, D), np.int8).tobytes() == wq.tobytes() and b.dl(bs, (B, D // 32)).tobytes() == wd.tobytes()


# ---- group 2 ---------------------------------------------------------------------------------
@case("halo_l2norm")
def _l2norm(b, name):
    rows, d = 9, 128
    x = synth.act("n.l2.x", rows, d)
    bx = b.up(x)
    b.run(name, (rows,), (128,), [B_(bx), U(d), F(EPS)])
    assert_rows_close(b.dl(bx, (rows, d)), b.orc.l2norm_rows(x.copy(), EPS), what=name)


@case("halo_gated_norm", "halo_gated_norm_h", "halo_gated_norm_hz", "halo_gated_norm_h128w", "halo_gated_norm_h128w_hh")
def _gated(b, name):
    rows, d = 24, 128
    o, z = synth.act("n.g.o", rows, d) * 2, synth.act("n.g.z", rows, d) * 3
    w = synth.gated_w("n.g.w", d)
    bw = b.up(w)
    for mode in (0, 1):
        if name == "halo_gated_norm":  # fp32, in place on o
            bo = b.up(o)
            b.run(name, (rows,), (256,), [B_(bo), B_(bw), B_(b.up(z)), U(d), F(EPS), U(mode)])
            assert_rows_close(b.dl(bo, (rows, d)), b.orc.gated_norm_rows(o.copy(), w, z, EPS, mode), what=f"{name} mode {mode}")
            continue
        hh = name.endswith("_hh")
        zh = hh or name.endswith("_hz")
        obits, ov = as16(o, "f16" if hh else "f32")
        zbits, zv = as16(z, "f16" if zh else "f32")
        by = b.new(rows * d * 2, 0)
        if "h128w" in name:  # one warp per row: rows is a parameter, the grid is rows / 8 blocks of 8 warps
            b.run(name, ((rows + 7) // 8,), (256,), [B_(b.up(obits)), B_(bw), B_(b.up(zbits)), B_(by), U(rows), F(EPS), U(mode)])
        else:
            b.run(name, (rows,), (128,), [B_(b.up(obits)), B_(bw), B_(b.up(zbits)), B_(by), U(d), F(EPS), U(mode)])
        got = b.dl(by, (rows, d), np.float16)
        want = b.orc.gated_norm_rows(ov.copy(), w, zv, EPS, mode)
        assert ulp16(got, want, "f16").max() <= 1, f"{name} mode {mode}"
        if name == "halo_gated_norm_h128w":  # the wave form equals the block form bit for bit
            by2 = b.new(rows * d * 2, 0)
            b.run("halo_gated_norm_h", (rows,), (128,), [B_(b.up(obits)), B_(bw), B_(b.up(zbits)), B_(by2), U(d), F(EPS), U(mode)])
            assert b.dl(by2, (rows, d), np.float16).tobytes() == got.tobytes(), "h128w differs from the block form"


# ---- group 3 ---------------------------------------------------------------------------------
def check_rope(got, want, x_in, rot, what):
    half = rot // 2
    bound = 1e-5 * np.maximum(np.maximum(np.abs(x_in[..., :half]), np.abs(x_in[..., half:rot])), 1e-30)
    assert np.all(np.abs(got[..., :half] - want[..., :half]) <= bound), what
    assert np.all(np.abs(got[..., half:rot] - want[..., half:rot]) <= bound), what
    assert got[..., rot:].tobytes() == x_in[..., rot:].tobytes(), what + " (dims beyond rot changed)"


@case("halo_rope_neox", "halo_rope_neox_rows", "halo_rope_neox_p", "halo_rope_neox_blocks", "halo_rope_neox_p_y")
def _rope(b, name):
    s = synth.FULL
    heads, hd, rot, th = 3, s.head_dim, s.rot, s.theta
    if name == "halo_rope_neox":
        x = synth.act("n.ro.x", 1, heads, hd)
        bx = b.up(x)
        b.run(name, (heads,), (64,), [B_(bx), U(hd), U(rot), U(262143), F(th)])
        check_rope(b.dl(bx, x.shape), b.orc.rope_rows(x.copy(), np.array([262143], np.uint32), rot, th), x, rot, name)
    elif name == "halo_rope_neox_rows":
        T, pos0 = 6, 4090
        x = synth.act("n.ro.rows", T, heads, hd)
        bx = b.up(x)
        b.run(name, (T * heads,), (64,), [B_(bx), U(hd), U(rot), U(pos0), U(heads), F(th)])
        check_rope(b.dl(bx, x.shape), b.orc.rope_rows(x.copy(), np.arange(pos0, pos0 + T, dtype=np.uint32), rot, th), x, rot, name)
    elif name == "halo_rope_neox_p":
        x = synth.act("n.ro.p", 1, heads, hd)
        bx, bp = b.up(x), b.up(np.array([9, 65537, 1, 1], np.uint32))
        b.run(name, (heads,), (64,), [B_(bx), B_(bp), U(hd), U(rot), U(1), U(3), F(th)])
        check_rope(b.dl(bx, x.shape), b.orc.rope_rows(x.copy(), np.array([65537 * 3], np.uint32), rot, th), x, rot, name)
    elif name == "halo_rope_neox_blocks":
        nb, b0, ratio = 5, 7, 128
        x = synth.act("n.ro.b", nb, 1, hd)
        bx = b.up(x)
        b.run(name, (nb,), (64,), [B_(bx), U(hd), U(rot), U(b0), U(ratio), F(th)])
        check_rope(b.dl(bx, x.shape), b.orc.rope_rows(x.copy(), ((b0 + np.arange(nb)) * ratio).astype(np.uint32), rot, th), x, rot, name)
    else:
        batch, stride, pstride = 4, heads * hd + 32, 16
        arena = synth.act("n.ro.y", batch * stride)
        prm = np.zeros((batch, pstride), np.uint32)
        prm[:, 1] = [5, 99999, 0, 262143]
        bx, bp = b.up(arena), b.up(prm)
        b.run(name, (heads, batch), (64,), [B_(bx), B_(bp), U(hd), U(rot), U(1), U(1), F(th), U(stride), U(pstride)])
        got, src = b.dl(bx, (batch, stride)), arena.reshape(batch, stride)
        for e in range(batch):
            xe = src[e, :heads * hd].reshape(1, heads, hd)
            check_rope(got[e, :heads * hd].reshape(1, heads, hd), b.orc.rope_rows(xe.copy(), prm[e:e + 1, 1], rot, th), xe, rot, f"{name} entry {e}")
            assert got[e, heads * hd:].tobytes() == src[e, heads * hd:].tobytes()


@case("halo_split_qgate", "halo_split_qgate_y")
def _split(b, name):
    heads, hd = 4, 64
    if name == "halo_split_qgate":
        rows = 3 * heads
        qg = synth.act("n.sp.qg", rows, 2, hd)
        bq, bg = b.new(rows * hd * 4), b.new(rows * hd * 4)
        b.run(name, (rows,), (256,), [B_(b.up(qg)), B_(bq), B_(bg), U(hd)])
        assert b.dl(bq, (rows, hd)).tobytes() == np.ascontiguousarray(qg[:, 0]).tobytes()
        assert b.dl(bg, (rows, hd)).tobytes() == np.ascontiguousarray(qg[:, 1]).tobytes()
    else:  # entry e (grid.y): q|gate rows at qg + e qg_stride, outputs at q / gate + e q_stride
        batch, qgs, qs = 3, heads * 2 * hd + 16, heads * hd + 8
        qg = synth.act("n.sp.y", batch, qgs)
        bq, bg = b.new(batch * qs * 4, 0), b.new(batch * qs * 4, 0)
        b.run(name, (heads, batch), (256,), [B_(b.up(qg)), B_(bq), B_(bg), U(hd), U(qgs), U(qs)])
        q, g = b.dl(bq, (batch, qs)), b.dl(bg, (batch, qs))
        for e in range(batch):
            rows = qg[e, :heads * 2 * hd].reshape(heads, 2, hd)
            assert q[e, :heads * hd].tobytes() == np.ascontiguousarray(rows[:, 0]).tobytes(), f"{name} q entry {e}"
            assert g[e, :heads * hd].tobytes() == np.ascontiguousarray(rows[:, 1]).tobytes(), f"{name} gate entry {e}"
            assert not q[e, heads * hd:].any() and not g[e, heads * hd:].any()


@case("halo_split_qgate_norm_rope", "halo_norm_rope_rows")
def _norm_rope(b, name):
    s = synth.FULL
    T, heads, hd, pos0 = 5, 4, s.head_dim, 300000
    w = 1 + synth.norm_w("n.nr.w", hd)
    pos = np.arange(pos0, pos0 + T, dtype=np.uint32)
    if name == "halo_split_qgate_norm_rope":
        qg = synth.act("n.nr.qg", T * heads, 2, hd)
        bq, bg = b.new(T * heads * hd * 4), b.new(T * heads * hd * 4)
        b.run(name, (T * heads,), (hd,), [B_(b.up(qg)), B_(bq), B_(bg), B_(b.up(w)), F(s.eps), U(s.rot), U(pos0), U(heads), F(s.theta)])
        x = np.ascontiguousarray(qg[:, 0])
        want = b.orc.rope_rows(b.orc.rmsnorm_rows(x.copy(), w, s.eps).reshape(T, heads, hd), pos, s.rot, s.theta)
        assert_rows_close(b.dl(bq, (T * heads, hd)), want.reshape(-1, hd), what=name)
        assert b.dl(bg, (T * heads, hd)).tobytes() == np.ascontiguousarray(qg[:, 1]).tobytes()
    else:
        x = synth.act("n.nr.x", T * heads, hd)
        bx, bc = b.up(x), b.new(x.nbytes, 0)
        b.run(name, (T * heads,), (256,), [B_(bx), B_(b.up(w)), F(s.eps), U(hd), U(s.rot), U(pos0), U(heads), F(s.theta), B_(bc)])
        want = b.orc.rope_rows(b.orc.rmsnorm_rows(x.copy(), w, s.eps).reshape(T, heads, hd), pos, s.rot, s.theta)
        got = b.dl(bx, (T * heads, hd))
        assert_rows_close(got, want.reshape(-1, hd), what=name)
        assert b.dl(bc, (T * heads, hd)).tobytes() == got.tobytes(), "cache row differs from the rotated row"


# ---- group 4 ---------------------------------------------------------------------------------
@case("halo_silu_mul", "halo_silu_mul_h", "halo_sigmoid_gate")
def _swiglu(b, name):
    n = 5 * 512 + 3
    g, up = synth.act("n.sw.g", n) * 4, synth.act("n.sw.u", n)
    grid = ((n + 255) // 256,)
    if name == "halo_silu_mul":
        bg = b.up(g)
        b.run(name, grid, (256,), [B_(bg), B_(b.up(up)), U(n)])
        close_elt(b.dl(bg, (n,)), b.orc.silu_mul(g.copy(), up), what=name)
    elif name == "halo_silu_mul_h":
        by = b.new(n * 2)
        b.run(name, grid, (256,), [B_(b.up(g)), B_(b.up(up)), B_(by), U(n)])
        assert ulp16(b.dl(by, (n,), np.float16), b.orc.silu_mul(g.copy(), up), "f16").max() <= 1, name
    else:  # x *= sigmoid(gate): the attention output gate (src/model/reference.cpp:360-363)
        bx = b.up(up)
        b.run(name, grid, (256,), [B_(bx), B_(b.up(g)), U(n)])
        close_elt(b.dl(bx, (n,)), (up * sigmoid_ref(b.orc, g)).astype(np.float32), what=name)


# ---- group 5 ---------------------------------------------------------------------------------
@case("halo_matvec_q8_0_embed", "halo_matvec_q8_0_embed_p", "halo_matvec_q8_0_embed_rows")
def _embed(b, name):
    s, vocab, T = synth.C1, 300, 9
    table = synth.q8_0_table("n.e.table", vocab, s.hidden)
    ids = synth.token_ids("n.e.ids", T, vocab)
    ids[0], ids[-1] = 0, vocab - 1
    want = b.orc.embed_q8_0_rows(table, ids, s.hidden)
    params = np.full((T, 16), 0xDEAD, np.uint32)
    params[:, 0] = ids
    bt, bp = b.up(table), b.up(params)
    grid_x = (s.hidden + 255) // 256
    if name == "halo_matvec_q8_0_embed":
        bo = b.new(s.hidden * 4)
        b.run(name, (grid_x,), (256,), [B_(bt), B_(bo), U(int(ids[4])), U(s.hidden), U64(s.q8_row_bytes)])
        assert b.dl(bo, (s.hidden,)).tobytes() == want[4].tobytes()
    elif name == "halo_matvec_q8_0_embed_p":
        bo = b.new(s.hidden * 4)
        b.run(name, (grid_x,), (256,), [B_(bt), B_(bo), B_(bp, 5 * 64), U(s.hidden), U64(s.q8_row_bytes)])
        assert b.dl(bo, (s.hidden,)).tobytes() == want[5].tobytes()
    else:
        bo = b.new(T * s.hidden * 4)
        b.run(name, (grid_x, T), (256,), [B_(bt), B_(bo), B_(bp), U(s.hidden), U64(s.q8_row_bytes)])
        assert b.dl(bo, (T, s.hidden)).tobytes() == want.tobytes()


# ---- hyper-connection residual -----------------------------------------------------------------
def hc_inputs(tag, T, hc, h, dt):
    res_bits, res = as16(synth.act(tag + ".res", T, hc, h), dt)
    out = synth.act(tag + ".out", T, h)
    inject = synth.act(tag + ".inj", T, hc) * 2
    w = (1 + 0.1 * synth.act(tag + ".w", hc, h)).astype(np.float32)
    return res_bits, res, out, inject, w


def check_hc_res(got, want, dt, what, mag):
    if dt == "f32":
        assert np.all(np.abs(got - want) <= 4e-7 * mag + 1e-30), what
    else:
        d = ulp16(as16(got, dt)[0], want, dt)
        assert d.max() <= 1 and (d == 0).mean() > 0.99, what


ROUND = {"f32": 0, "bf16": 1, "f16": 2}
DT16 = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16}


@case("halo_hc_combine_norm_rows", "halo_hc_combine_norm_rows_r16", "halo_hc_combine_norm_rows_rb",
      "halo_hc_combine_norm_rows_q8")
def _hc_rows(b, name):
    q8 = name.endswith("_q8")
    dt = "f32" if q8 else SUFFIX[name[len("halo_hc_combine_norm_rows"):]]
    T, hc, h = 6, 4, 256
    res_bits, res, out, inject, w = hc_inputs("n.hcr." + dt, T, hc, h, dt)
    br, by, by16, brs = b.up(res_bits), b.new(T * hc * h * 4), b.new(T * hc * h * 2), b.new(T * hc * 4)
    args = [B_(br), B_(b.up(out)), B_(b.up(inject)), B_(b.up(w)), B_(by), B_(by16), U(hc), U(h), F(EPS), Arg.Null, Arg.Null,
            U(0), B_(brs), U(T if q8 else 0)]
    if q8:
        byq, byd = b.new(T * hc * h), b.new(T * hc * h // 32 * 4)
        args += [B_(byq), B_(byd)]
    b.run(name, (T * hc,), (256,), args)
    got_res = from16(b.dl(br, (T, hc, h), DT16[dt]), dt)
    want_res = res.copy()
    b.orc.hc_combine_norm(want_res, out, inject, w, EPS, ROUND[dt])
    check_hc_res(got_res, want_res, dt, name + " residual", np.abs(res) + 2 * np.abs(out)[:, None, :])
    want_y = b.orc.hc_combine_norm(got_res.copy(), None, None, w, EPS, 0)  # two-stage: the norm of what the GPU stored
    got_y = b.dl(by, (T, hc, h))
    assert_rows_close(got_y.reshape(-1, h), want_y.reshape(-1, h), what=name + " y")
    h16 = b.dl(by16, (T * hc * h,), np.float16)
    if q8:  # the fp16 copy and the int8 copy are K-blocked [hc h / 64][T][64]
        h16 = h16.reshape(hc * h // 64, T, 64).transpose(1, 0, 2)
        wq, wd = b.orc.quantize_i8_rows(got_y.reshape(T, hc * h))
        assert b.dl(byq, (hc * h // 64, T, 64), np.int8).tobytes() == wq.reshape(T, hc * h // 64, 64).transpose(1, 0, 2).tobytes()
        assert b.dl(byd, (hc * h // 32, T)).tobytes() == np.ascontiguousarray(wd.T).tobytes()
    assert np.array_equal(h16.reshape(T, hc, h), got_y.astype(np.float16)), name + " fp16 copy"
    rs = b.dl(brs, (T * hc,))
    assert np.allclose(rs, 1 / np.sqrt((got_res.astype(np.float64) ** 2).mean(axis=2).reshape(-1) + EPS), rtol=2e-6)


@case("halo_hc_combine_norm_tok", "halo_hc_combine_norm_tok_r16", "halo_hc_combine_norm_tok_rb")
def _hc_tok(b, name):
    dt = SUFFIX[name[len("halo_hc_combine_norm_tok"):]]
    T, hc, h = 5, 4, 2048
    res_bits, res, out, inject, w = hc_inputs("n.hct." + dt, T, hc, h, dt)
    br, by16 = b.up(res_bits), b.new(T * hc * h * 2)
    b.run(name, (T,), (256,), [B_(br), B_(b.up(out)), B_(b.up(inject)), B_(b.up(w)), B_(by16), U(h), F(EPS), Arg.Null,
                               Arg.Null, U(0), Arg.Null, U(0)])
    got_res = from16(b.dl(br, (T, hc, h), DT16[dt]), dt)
    want_res = res.copy()
    b.orc.hc_combine_norm(want_res, out, inject, w, EPS, ROUND[dt])
    check_hc_res(got_res, want_res, dt, name + " residual", np.abs(res) + 2 * np.abs(out)[:, None, :])
    want_y = b.orc.hc_combine_norm(got_res.copy(), None, None, w, EPS, 0)
    assert ulp16(b.dl(by16, (T, hc, h), np.float16), want_y, "f16").max() <= 1, name + " y16"


@case("halo_hc_combine_norm_tok_moe", "halo_hc_combine_norm_tok_moe_r16", "halo_hc_combine_norm_tok_moe_rb",
      "halo_hc_combine_norm_tok_moev", "halo_hc_combine_norm_tok_moev_r16", "halo_hc_combine_norm_tok_moev_rb")
def _hc_tok_moe(b, name):
    dt = "f16" if name.endswith("_r16") else "bf16" if name.endswith("_rb") else "f32"
    T, hc, h, k = 4, 4, 2048, 10
    res_bits, res, _, inject, w = hc_inputs("n.hcm." + dt, T, hc, h, dt)
    yp = synth.act("n.hcm.yp", T * k, h).astype(np.float16)
    pos = synth.rng("n.hcm.pos").permutation(T * k).reshape(T, k).astype(np.uint32)
    mw = synth.rng("n.hcm.mw").random((T, k), dtype=np.float32)
    sx, sg = synth.act("n.hcm.sx", T, h), synth.act("n.hcm.sg", T)
    br, by16 = b.up(res_bits), b.new(T * hc * h * 2)
    b.run(name, (T,), (256,), [B_(br), B_(b.up(yp)), B_(b.up(pos)), B_(b.up(mw)), B_(b.up(sx)), B_(b.up(sg)), U(k),
                               B_(b.up(inject)), B_(b.up(w)), B_(by16), U(h), F(EPS), Arg.Null, Arg.Null, U(0), Arg.Null, U(0)])
    out = b.orc.moe_combine(yp.astype(np.float32), pos, mw, sx, sg)
    got_res = from16(b.dl(br, (T, hc, h), DT16[dt]), dt)
    want_res = res.copy()
    b.orc.hc_combine_norm(want_res, out, inject, w, EPS, ROUND[dt])
    check_hc_res(got_res, want_res, dt, name + " residual", np.abs(res) + 2 * np.abs(out)[:, None, :])
    want_y = b.orc.hc_combine_norm(got_res.copy(), None, None, w, EPS, 0)
    assert ulp16(b.dl(by16, (T, hc, h), np.float16), want_y, "f16").max() <= 1, name + " y16"


@case("halo_hc_combine", "halo_hc_combine_rows", "halo_hc_combine_rows_r16", "halo_hc_combine_rows_rb")
def _hc_combine(b, name):
    single = name == "halo_hc_combine"
    dt = "f32" if single else SUFFIX[name[len("halo_hc_combine_rows"):]]
    T, hc, h = (1 if single else 5), 4, 320
    res_bits, res, out, inject, _ = hc_inputs("n.hcc." + dt, T, hc, h, dt)
    br = b.up(res_bits)
    args = [B_(br), B_(b.up(out)), B_(b.up(inject)), U(hc), U(h)] + ([] if single else [U(T)])
    b.run(name, ((T * hc * h + 255) // 256,), (256,), args)
    want = res.copy()
    b.orc.hc_combine_norm(want, out, inject, np.ones((hc, h), np.float32), EPS, ROUND[dt])
    check_hc_res(from16(b.dl(br, (T, hc, h), DT16[dt]), dt), want, dt, name, np.abs(res) + 2 * np.abs(out)[:, None, :])


@case("halo_broadcast", "halo_broadcast_rows", "halo_broadcast_rows_r16", "halo_broadcast_rows_rb")
def _broadcast(b, name):
    single = name == "halo_broadcast"
    dt = "f32" if single else SUFFIX[name[len("halo_broadcast_rows"):]]
    T, hc, h = (1 if single else 4), 4, 264
    x = synth.act("n.bc.x", T, h)
    br = b.new(T * hc * h * (4 if dt == "f32" else 2), 0)
    b.run(name, ((T * hc * h + 255) // 256,), (256,), [B_(br), B_(b.up(x)), U(hc), U(h)] + ([] if single else [U(T)]))
    want = as16(np.broadcast_to(x[:, None, :], (T, hc, h)).copy(), dt)[0]
    assert b.dl(br, (T, hc, h), DT16[dt]).tobytes() == want.tobytes(), name


@case("halo_hc_mix", "halo_hc_mix_rows")
def _hc_mix(b, name):
    single = name == "halo_hc_mix"
    T, hc, h = (1 if single else 5), 4, 256
    xn, gate = synth.act("n.mix.xn", T, hc, h), synth.act("n.mix.g", T, hc, h) * 2
    bm = b.new(T * h * 4)
    b.run(name, ((T * h + 255) // 256,), (256,), [B_(b.up(xn)), B_(b.up(gate)), B_(bm), U(hc), U(h)] + ([] if single else [U(T)]))
    got, want = b.dl(bm, (T, h)), b.orc.hc_mix(xn, gate)
    assert np.all(np.abs(got - want) <= 1e-5 * np.abs(xn).sum(axis=1) / hc + 1e-30), name


@case("halo_axpy_sigmoid", "halo_axpy_sigmoid_rows")
def _axpy_sigmoid(b, name):
    single = name == "halo_axpy_sigmoid"
    T, n = (1 if single else 6), 520
    y, x, g = synth.act("n.as.y", T, n), synth.act("n.as.x", T, n), synth.act("n.as.g", T) * 3
    by = b.up(y)
    b.run(name, ((T * n + 255) // 256,), (256,), [B_(by), B_(b.up(x)), B_(b.up(g)), U(n)] + ([] if single else [U(T)]))
    want = y + sigmoid_ref(b.orc, g)[:, None] * x
    assert np.all(np.abs(b.dl(by, (T, n)) - want) <= 4e-7 * (np.abs(y) + np.abs(x)) + 1e-30), name


@case("halo_inject_reduce")
def _inject_reduce(b, name):
    T, hc, irows = 7, 4, 5
    ip = synth.act("n.ir.ip", T, hc, irows)
    bo = b.new(T * irows * 4)
    b.run(name, ((T * irows + 255) // 256,), (256,), [B_(b.up(ip)), B_(bo), U(hc), U(irows), U(T)])
    want = ip[:, 0].copy()
    for s_ in range(1, hc):
        want = want + ip[:, s_]  # streams summed in order
    assert b.dl(bo, (T, irows)).tobytes() == want.astype(np.float32).tobytes(), name


@case("halo_res_to_f32_r16", "halo_res_to_f32_rb")
def _res_to_f32(b, name):
    dt = "f16" if name.endswith("_r16") else "bf16"
    n = 1000
    bits, vals = as16(synth.act("n.r2f.x", n) * 5, dt)
    by = b.new(n * 4)
    b.run(name, ((n + 255) // 256,), (256,), [B_(by), B_(b.up(bits)), U(n)])
    assert b.dl(by, (n,)).tobytes() == vals.astype(np.float32).tobytes(), name


@case("halo_hc_norm_scales", "halo_hc_norm_scales_u")
def _hc_norm_scales(b, name):
    rows, h = 12, 2048
    res = synth.act("n.ns.res", rows, h) * 2
    bs = b.new(rows * 4)
    b.run(name, (rows,), (256,), [B_(b.up(res)), B_(bs), U(h), F(EPS)])
    want = 1 / np.sqrt((res.astype(np.float64) ** 2).mean(axis=1) + EPS)
    assert np.allclose(b.dl(bs, (rows,)), want, rtol=2e-6), name


# ---- Gated DeltaNet conv ---------------------------------------------------------------------
def conv_inputs(tag, T, C, kern):
    x = synth.act(tag + ".x", T, C)
    state = np.ascontiguousarray(synth.act(tag + ".st", max(kern - 1, 1), C)[:kern - 1])
    w = (synth.act(tag + ".w", C, kern) * 0.5).astype(np.float32)
    return x, state, w


def check_conv(got, want, d, l2, what):
    if l2:
        assert_rows_close(got[:, :l2].reshape(-1, d), want[:, :l2].reshape(-1, d), what=what + " q/k")
    if l2 < got.shape[1]:
        assert_rows_close(got[:, l2:], want[:, l2:], what=what + " v")


@case("halo_conv_l2norm_prefill", "halo_conv_l2norm_prefill8", "halo_conv_l2norm_prefill8_h", "halo_conv_l2norm_prefill8_hh")
def _conv_prefill(b, name):
    T, C, l2, d, kern = 13, 1024, 512, 128, 4
    x, state, w = conv_inputs("n.cv", T, C, kern)
    idt = "f16" if name.endswith(("_h", "_hh")) else "f32"
    odt = "f16" if name.endswith("_hh") else "f32"
    xbits, xv = as16(x, idt)
    bo = b.new(T * C * (2 if odt == "f16" else 4))
    if name == "halo_conv_l2norm_prefill":
        b.run(name, (C // d, T), (d,), [B_(b.up(xbits)), B_(b.up(state)), B_(b.up(w)), B_(bo), U(C), U(kern), U(l2), F(EPS)])
    else:
        b.run(name, (C // d, (T + 7) // 8), (d,), [B_(b.up(xbits)), B_(b.up(state)), B_(b.up(w)), B_(bo), U(C), U(T), U(l2), F(EPS)])
    want = b.orc.conv_l2norm(xv, state.copy(), w, l2, d, EPS)
    if odt == "f16":
        assert ulp16(b.dl(bo, (T, C), np.float16), want, "f16").max() <= 1, name
    else:
        check_conv(b.dl(bo, (T, C)), want, d, l2, name)


@case("halo_conv_state_advance", "halo_conv_state_advance_h")
def _conv_advance(b, name):
    C, kern = 512, 4
    idt = "f16" if name.endswith("_h") else "f32"
    for T in (9, 2):  # a chunk shorter than the state keeps older rows of the previous state
        x, state, _ = conv_inputs(f"n.cva{T}", T, C, kern)
        xbits, xv = as16(x, idt)
        bs = b.up(state)
        b.run(name, ((C + 255) // 256,), (256,), [B_(b.up(xbits)), B_(bs), U(C), U(kern), U(T)])
        want = np.concatenate([state, xv])[-(kern - 1):]
        assert b.dl(bs, (kern - 1, C)).tobytes() == want.astype(np.float32).tobytes(), f"{name} T={T}"


@case("halo_conv_step", "halo_conv_l2norm", "halo_conv_l2norm_y")
def _conv_step(b, name):
    C, l2, d, kern = 512, 256, 128, 4
    if name == "halo_conv_l2norm_y":
        import torch
        B = 3
        x, _, w = conv_inputs("n.cvy", B, C, kern)
        states = [np.ascontiguousarray(synth.act(f"n.cvy.s{e}", 3, C)) for e in range(B)]
        d_states = [torch.from_numpy(s_.copy()).to("cuda:0") for s_ in states]
        tab = np.array([[0, t.data_ptr()] for t in d_states], np.uint64)
        bo = b.new(B * C * 4)
        torch.cuda.synchronize()
        b.run(name, (C // d, B), (d,), [B_(b.up(x)), B_(b.up(tab)), U(2), U(1), B_(b.up(w)), B_(bo), U(C), U(kern), U(l2), F(EPS), U(C)])
        got = b.dl(bo, (B, C))
        for e in range(B):
            hist = states[e].copy()
            check_conv(got[e:e + 1], b.orc.conv_l2norm(x[e:e + 1], hist, w, l2, d, EPS), d, l2, f"{name} entry {e}")
            assert np.array_equal(d_states[e].cpu().numpy(), hist), f"{name} state {e}"
        return
    x, state, w = conv_inputs("n.cvs", 1, C, kern)
    bs, bo = b.up(state), b.new(C * 4)
    if name == "halo_conv_step":
        b.run(name, ((C + 255) // 256,), (256,), [B_(b.up(x)), B_(bs), B_(b.up(w)), B_(bo), U(C), U(kern)])
        l2 = 0
    else:
        b.run(name, (C // d,), (d,), [B_(b.up(x)), B_(bs), B_(b.up(w)), B_(bo), U(C), U(kern), U(l2), F(EPS)])
    hist = state.copy()
    check_conv(b.dl(bo, (1, C)), b.orc.conv_l2norm(x, hist, w, l2, d, EPS), d, l2, name)
    assert np.array_equal(b.dl(bs, (kern - 1, C)), hist), name + " state"


# ---- row copies ------------------------------------------------------------------------------
@case("halo_copy", "halo_f16_rows", "halo_copy_at", "halo_copy_at_h", "halo_copy_at_y")
def _copies(b, name):
    n, rows = 520, 6
    src = synth.act("n.cp.src", n)
    params = np.zeros(16, np.uint32)
    params[1] = 4
    grid = ((n + 255) // 256,)
    if name == "halo_copy":
        bd = b.new(n * 4)
        b.run(name, grid, (256,), [B_(bd), B_(b.up(src)), U(n)])
        assert b.dl(bd, (n,)).tobytes() == src.tobytes()
    elif name == "halo_f16_rows":
        bd = b.new(n * 2)
        b.run(name, grid, (256,), [B_(b.up(src)), B_(bd), U(n)])
        assert np.array_equal(b.dl(bd, (n,), np.float16), src.astype(np.float16))
    elif name in ("halo_copy_at", "halo_copy_at_h"):
        np_dt = np.float16 if name.endswith("_h") else np.float32
        cache = np.full((rows, n), 7.0, np_dt)
        bc = b.up(cache)
        b.run(name, grid, (256,), [B_(bc), B_(b.up(src)), B_(b.up(params)), U(1), U(n), U(n)])
        cache[4] = src.astype(np_dt)
        assert np.array_equal(b.dl(bc, (rows, n), np_dt), cache), name
    else:
        import torch
        B, src_stride, pstride = 3, n + 8, 16
        srcs = synth.act("n.cp.y", B, src_stride)
        caches = [torch.full((rows, n), -1.0, device="cuda:0") for _ in range(B)]
        pos = [4, 0, 5]
        prm = np.zeros((B, pstride), np.uint32)
        prm[:, 1] = pos
        tab = np.array([[0, 0, c.data_ptr(), 0] for c in caches], np.uint64)
        torch.cuda.synchronize()
        b.run(name, (grid[0], B), (256,), [B_(b.up(tab)), U(4), U(2), B_(b.up(srcs)), B_(b.up(prm)), U(1), U(n), U(n), U(src_stride), U(pstride)])
        b.dev.synchronize()
        for e in range(B):
            want = np.full((rows, n), -1.0, np.float32)
            want[pos[e]] = srcs[e, :n]
            assert caches[e].cpu().numpy().tobytes() == want.tobytes(), f"{name} entry {e}"


@case("halo_scale_silu", "halo_scale_silu_h")
def _scale_silu(b, name):
    n = 777
    x = synth.act("n.ss.x", n) * 4
    want = silu_ref(b.orc, (x * np.float32(0.25)).astype(np.float32))
    bx = b.up(x)
    if name == "halo_scale_silu":
        b.run(name, ((n + 255) // 256,), (256,), [B_(bx), F(0.25), U(n)])
        close_elt(b.dl(bx, (n,)), want, what=name)
    else:
        by = b.new(n * 2)
        b.run(name, ((n + 255) // 256,), (256,), [B_(bx), B_(by), F(0.25), U(n)])
        assert ulp16(b.dl(by, (n,), np.float16), want, "f16").max() <= 1, name


# ---- MoE combine -------------------------------------------------------------------------------
@case("halo_moe_combine_grouped", "halo_moe_combine_shared", "halo_moe_combine", "halo_moe_combine_u", "halo_axpy_slot")
def _moe(b, name):
    T, k, n = 5, 10, 2048
    if name in ("halo_moe_combine_grouped", "halo_moe_combine_shared"):
        yp = synth.act("n.moe.yp", T * k, n).astype(np.float16)
        pos = synth.rng("n.moe.pos").permutation(T * k).reshape(T, k).astype(np.uint32)
        mw = synth.rng("n.moe.mw").random((T, k), dtype=np.float32)
        sx, sg = synth.act("n.moe.sx", T, n), synth.act("n.moe.sg", T)
        bo = b.new(T * n * 4)
        if name.endswith("grouped"):
            b.run(name, ((n + 255) // 256, T), (256,), [B_(b.up(yp)), B_(b.up(pos)), B_(b.up(mw)), B_(bo), U(k), U(n)])
            assert b.dl(bo, (T, n)).tobytes() == b.orc.moe_combine(yp.astype(np.float32), pos, mw).tobytes(), name
        else:
            b.run(name, ((n + 255) // 256, T), (256,), [B_(b.up(yp)), B_(b.up(pos)), B_(b.up(mw)), B_(b.up(sx)), B_(b.up(sg)), B_(bo), U(k), U(n)])
            routed = b.orc.moe_combine(yp.astype(np.float32), pos, mw)
            want = b.orc.moe_combine(yp.astype(np.float32), pos, mw, sx, sg)
            assert np.all(np.abs(b.dl(bo, (T, n)) - want) <= 4e-7 * (np.abs(routed) + np.abs(sx)) + 1e-30), name
    elif name in ("halo_moe_combine", "halo_moe_combine_u"):
        part, wts = synth.act("n.moe.part", k, n), synth.rng("n.moe.w1").random(k, dtype=np.float32)
        bo = b.new(n * 4)
        b.run(name, ((n + 255) // 256,), (256,), [B_(b.up(part)), B_(b.up(wts)), B_(bo), U(k), U(n)])
        want = b.orc.moe_combine(part, np.arange(k, dtype=np.uint32).reshape(1, k), wts.reshape(1, k))[0]  # slots in order
        assert b.dl(bo, (n,)).tobytes() == want.tobytes(), name
    else:
        y, x, wts = synth.act("n.moe.y", n), synth.act("n.moe.x", n), synth.rng("n.moe.w2").random(k, dtype=np.float32)
        by = b.up(y)
        b.run(name, ((n + 255) // 256,), (256,), [B_(by), B_(b.up(x)), B_(b.up(wts)), U(3), U(n)])
        assert b.dl(by, (n,)).tobytes() == (y + wts[3] * x).astype(np.float32).tobytes(), name


# ---- the table is complete, and every case passes ---------------------------------------------------
def test_every_kernel_name_has_a_case():
    names = lib().kernel_names()
    assert len(names) == len(set(names))
    missing = [n for n in names if n not in CASES]
    assert not missing, f"kernel names without a by-name parity case: {missing}"
    unknown = [n for n in CASES if n not in names]
    assert not unknown, f"cases for names the library does not export: {unknown}"


@pytest.fixture(scope="module")
def box(orc):
    return Box(Device.create(0), orc)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(CASES))
def test_launch_by_name(box, name):
    CASES[name](box, name)
    box.dev.synchronize()
