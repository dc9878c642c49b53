"""Parity of the hyper-connection residual kernels with the CPU oracle, through the C ABI (GPU only).

The oracle repeats ReferenceModel::HcCombine / GroupedNorm / HcMix / Moe (src/model/reference.cpp:151-202,
558-578) around the reference's own scalar operators. Tolerances: the combined residual within 4e-7
relative in fp32 (the scatter weight 2 sigmoid(inject / hc) comes from the device's expf, 1-2 ulp from
libm's) and within 1 ulp of its 16-bit storage type; with zero inject logits (weight exactly 1) the
residual is bit-exact. The normalized outputs are checked two-stage, as the reference checks its fused
kernels (tests/gpu/quant_gpu_test.cpp:2428-2494): against the oracle's grouped norm of the residual the
GPU stored, fp32 within 1e-5, bf16 within 1 ulp; int8 copies and inject_reduce bit-exact on the GPU's own y.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_bf16_within_1ulp, assert_rows_close
from halo_flash_b200 import HaloError, lib, ops, synth
from halo_flash_b200.device import Arg, Device

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
EPS = 1e-6
TDT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
ROUND = {"f32": 0, "bf16": 1, "f16": 2}


def to_dev(a, dtype="f32"):
    if dtype == "bf16":
        return torch.from_numpy(oracle.bf16_bits(a).view(np.int16)).to(DEV).view(torch.bfloat16).reshape(a.shape)
    if dtype == "f16":
        return torch.from_numpy(a.astype(np.float16)).to(DEV)
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def to_f32(t):
    return t.detach().float().cpu().numpy()


def rounded(a, dtype):
    if dtype == "bf16":
        return oracle.round_bf16(a)
    if dtype == "f16":
        return a.astype(np.float16).astype(np.float32)
    return a.astype(np.float32)


def ulps16(got, want, dtype):
    """Distance in units of the 16-bit type between two arrays of representable values."""
    if dtype == "bf16":
        a, b = oracle.bf16_bits(got).astype(np.int32), oracle.bf16_bits(want).astype(np.int32)
    else:
        a, b = got.astype(np.float16).view(np.uint16).astype(np.int32), want.astype(np.float16).view(np.uint16).astype(np.int32)
    order = lambda v: np.where(v & 0x8000, 0x8000 - (v & 0x7FFF) - 1, 0x8000 + v)
    return np.abs(order(a) - order(b))


def inputs(tag, T, hc, h, rdt, odt):
    res = rounded(synth.act(tag + ".res", T, hc, h), rdt)
    out = rounded(synth.act(tag + ".out", T, h), odt)
    inject = synth.act(tag + ".inj", T, hc) * 2
    w = (1 + 0.1 * synth.act(tag + ".w", hc, h)).astype(np.float32)
    return res, out, inject, w


def check_res(got, want, rdt, what, mag=None):
    """mag: |res| + 2 |out| of the inputs, the scale of the two terms whose sum may cancel."""
    if rdt == "f32":
        assert np.all(np.abs(got - want) <= 4e-7 * (np.abs(want) if mag is None else mag) + 1e-30), what
    else:
        d = ulps16(got, want, rdt)
        assert d.max() <= 1 and (d == 0).mean() > 0.995, what


def check_y(y, want, what):
    if y.dtype == torch.float32:
        assert_rows_close(to_f32(y).reshape(-1, want.shape[-1]), want.reshape(-1, want.shape[-1]), what=what)
    elif y.dtype == torch.bfloat16:
        assert_bf16_within_1ulp(y.view(torch.int16).cpu().numpy().view(np.uint16), want, what=what)
    else:
        assert ulps16(to_f32(y), want.astype(np.float16).astype(np.float32), "f16").max() <= 1, what


SHAPES = [(7, 4, 256), (5, 4, 64), (3, 4, 2048), (3, 4, 2560), (6, 2, 256), (5, 3, 96), (4, 1, 512), (9, 4, 40)]


@pytest.mark.parametrize("T,hc,h", SHAPES)
@pytest.mark.parametrize("rdt,odt,ydt", [("f32", "f32", "f32"), ("bf16", "f32", "f32"), ("f16", "f32", "f32"),
                                         ("bf16", "bf16", "bf16"), ("f16", "f16", "f16"), ("bf16", "f16", "f32")])
@pytest.mark.parametrize("row_level", [0, 1])
def test_hc_combine_norm(orc, T, hc, h, rdt, odt, ydt, row_level):
    if row_level and hc != 4:
        pytest.skip("only hc = 4 has a token-level shape to switch off")
    res, out, inject, w = inputs(f"t.hc.{T}.{hc}.{h}", T, hc, h, rdt, odt)
    d_res, d_out, d_inj, d_w = to_dev(res, rdt), to_dev(out, odt), to_dev(inject), to_dev(w)
    y = torch.full((T, hc, h), float("nan"), device=DEV, dtype=TDT[ydt])
    rscale = torch.empty(T, hc, device=DEV)
    lib().tune("hc_row_level", row_level)
    try:
        ops.hc_combine_norm(d_res, d_out, d_inj, d_w, EPS, y=y, rscale=rscale)
    finally:
        lib().tune("hc_row_level", 0)
    want_res = res.copy()
    orc.hc_combine_norm(want_res, out, inject, w, EPS, ROUND[rdt])
    got_res = to_f32(d_res)
    check_res(got_res, want_res, rdt, "combined residual", np.abs(res) + 2 * np.abs(out)[:, None, :])
    # stage two: the grouped norm of what the GPU stored
    stored = got_res.copy()
    want_y = orc.hc_combine_norm(stored, None, None, w, EPS, 0)
    check_y(y, want_y, "grouped norm")
    ms = (got_res.astype(np.float64) ** 2).mean(axis=2)
    assert np.allclose(to_f32(rscale), 1 / np.sqrt(ms + EPS), rtol=2e-6)


def test_zero_inject_logits_make_a_plain_add(orc):
    """2 sigmoid(0 / hc) is exactly 1: the combine is a residual add into every stream, bit for bit."""
    T, hc, h = 33, 4, 2048
    res, out, _, w = inputs("t.hc.zero", T, hc, h, "bf16", "bf16")
    d_res = to_dev(res, "bf16")
    y = torch.empty(T, hc, h, device=DEV, dtype=torch.bfloat16)
    ops.hc_combine_norm(d_res, to_dev(out, "bf16"), torch.zeros(T, hc, device=DEV), to_dev(w), EPS, y=y)
    want = oracle.round_bf16(res + out[:, None, :])
    assert np.array_equal(oracle.bf16_bits(to_f32(d_res)), oracle.bf16_bits(want))
    res32 = synth.act("t.hc.zero32", T, hc, h)
    d32 = to_dev(res32)
    ops.hc_combine_rows(d32, to_dev(out), torch.zeros(T, hc, device=DEV))
    assert np.array_equal(to_f32(d32), res32 + out[:, None, :])


@pytest.mark.parametrize("T,hc,h,irows", [(6, 4, 256, 4), (5, 4, 2048, 8), (4, 4, 2560, 3), (7, 2, 128, 1)])
def test_hc_side_outputs(orc, T, hc, h, irows):
    """fp16 copy (row-major and K-blocked), int8 K-blocked copy, inject partial products."""
    res, out, inject, w = inputs(f"t.hc.side.{h}", T, hc, h, "f32", "f32")
    iw = synth.act(f"t.hc.iw.{h}", irows, hc * h) * 0.05
    Tk = T + 3  # the K-blocked buffers are laid out for a longer chunk than the rows written
    for blocked in (0, Tk):
        d_res = to_dev(res)
        y = torch.empty(T, hc, h, device=DEV)
        y16 = torch.zeros((hc * h // 64, Tk, 64) if blocked else (T, hc, h), device=DEV, dtype=torch.float16)
        yq = torch.zeros(hc * h // 64, Tk, 64, device=DEV, dtype=torch.int8)
        yd = torch.zeros(hc * h // 32, Tk, device=DEV)
        ipart = torch.full((T, hc, irows), float("nan"), device=DEV)
        ops.hc_combine_norm(d_res, to_dev(out), to_dev(inject), to_dev(w), EPS, y=y, y16=y16, y16_tokens=blocked,
                            iw=to_dev(iw), ipart=ipart, yq=yq if blocked else None, yd=yd if blocked else None)
        gy = to_f32(y)
        flat = gy.reshape(T, hc * h)
        if blocked:
            got16 = to_f32(y16).transpose(1, 0, 2).reshape(Tk, hc * h)[:T]
        else:
            got16 = to_f32(y16).reshape(T, hc * h)
        assert np.array_equal(got16, flat.astype(np.float16).astype(np.float32)), "fp16 copy = half_rne(y)"
        if blocked:
            blocks = flat.reshape(T, -1, 32)
            scale = (np.abs(blocks).max(axis=2) / np.float32(127.0)).astype(np.float32)
            with np.errstate(divide="ignore", invalid="ignore"):
                q = np.where(scale[..., None] > 0, np.rint(blocks / scale[..., None]), 0).astype(np.int8)
            gq = yq.cpu().numpy().transpose(1, 0, 2).reshape(Tk, hc * h)[:T]
            gd = yd.cpu().numpy().T[:T]
            assert np.array_equal(gd, scale) and np.array_equal(gq, q.reshape(T, hc * h)), "int8 copy"
        # partial products: their sum over the streams is the inject projection of y
        inj = torch.empty(T, irows, device=DEV)
        ops.inject_reduce(ipart, inj)
        gp = to_f32(ipart)
        seq = np.zeros((T, irows), np.float32)
        for s in range(hc):
            seq = seq + gp[:, s, :]
        assert np.array_equal(to_f32(inj), seq), "inject_reduce adds the streams in order"
        want = orc.hc_inject(flat, iw)
        bound = np.abs(flat[:, None, :] * iw[None, :, :]).sum(axis=2)
        assert np.all(np.abs(to_f32(inj) - want) <= 1e-5 * bound + 1e-30), "inject partial products"


@pytest.mark.parametrize("h,k,rdt,ypdt,sxdt", [(2048, 10, "f32", "f16", "f32"), (2560, 10, "f32", "f16", "f32"),
                                               (256, 2, "bf16", "f16", "f32"), (2048, 10, "bf16", "bf16", "bf16")])
def test_hc_combine_with_the_expert_sum(orc, h, k, rdt, ypdt, sxdt):
    T, hc = 6, 4
    ydt = "bf16" if ypdt == "bf16" else "f32"  # the all-bf16 engine form, or the reference's fp32 outputs
    res, _, inject, w = inputs(f"t.hc.moe.{h}", T, hc, h, rdt, "f32")
    yp = rounded(synth.act(f"t.hc.yp.{h}", T * k, h), ypdt)
    pos = synth.rng(f"t.hc.pos.{h}").permutation(T * k).reshape(T, k).astype(np.uint32)
    mw = synth.rng(f"t.hc.mw.{h}").random((T, k), dtype=np.float32)
    sx = rounded(synth.act(f"t.hc.sx.{h}", T, h), sxdt)
    sg = synth.act(f"t.hc.sg.{h}", T)
    want_out = orc.moe_combine(yp, pos, mw, sx, sg)
    args = (to_dev(yp, ypdt), torch.from_numpy(pos.view(np.int32)).to(DEV), to_dev(mw), to_dev(sx, sxdt), to_dev(sg))
    # zero residual and zero logits: the stored residual IS the expert sum
    z = torch.zeros(T, hc, h, device=DEV, dtype=TDT[rdt])
    y = torch.empty(T, hc, h, device=DEV, dtype=TDT[ydt])
    ops.hc_combine_norm_moe(z, *args, torch.zeros(T, hc, device=DEV), to_dev(w), EPS, y=y)
    gs = np.float32(1) / (np.float32(1) + np.exp(-sg, dtype=np.float32))
    got = to_f32(z)
    tol = 3e-7 * (np.abs(want_out) + np.abs(gs[:, None] * sx))  # sigmoid(sg) from the device's expf
    for s in range(hc):
        if rdt == "f32":
            assert np.all(np.abs(got[:, s] - want_out) <= tol + 1e-30), "expert sum"
        else:
            assert ulps16(got[:, s], rounded(want_out, rdt), rdt).max() <= 1, "expert sum"
    # the full op against the oracle chain
    for row_level in (0, 1):
        d_res = to_dev(res, rdt)
        y16 = torch.empty(T, hc, h, device=DEV, dtype=torch.float16)
        rscale = torch.empty(T, hc, device=DEV)
        lib().tune("hc_row_level", row_level)
        try:
            ops.hc_combine_norm_moe(d_res, *args, to_dev(inject), to_dev(w), EPS, y16=y16, rscale=rscale)
        finally:
            lib().tune("hc_row_level", 0)
        want_res = res.copy()
        orc.hc_combine_norm(want_res, want_out, inject, w, EPS, ROUND[rdt])
        got_res = to_f32(d_res)
        if rdt == "f32":
            assert np.all(np.abs(got_res - want_res) <= 1e-6 * (np.abs(want_res) + np.abs(want_out)[:, None, :]) + 1e-30)
        else:
            check_res(got_res, want_res, rdt, "residual after the expert sum")
        want_y = orc.hc_combine_norm(got_res.copy(), None, None, w, EPS, 0)
        assert ulps16(to_f32(y16), want_y.astype(np.float16).astype(np.float32), "f16").max() <= 1


@pytest.mark.parametrize("T,hc,h", [(5, 4, 256), (3, 4, 2048), (4, 3, 100), (2, 2, 2560)])
def test_stream_elementwise_ops(orc, T, hc, h):
    res, out, inject, _ = inputs(f"t.hc.elt.{h}", T, hc, h, "f32", "f32")
    for rdt in ("f32", "bf16", "f16"):
        r0 = rounded(res, rdt)
        d = to_dev(r0, rdt)
        ops.hc_combine_rows(d, to_dev(out), to_dev(inject))
        a = np.array([[2 * orc._call("orc_sigmoid", float(np.float32(v) / np.float32(hc))) for v in row] for row in inject],
                     np.float32)
        want = rounded(r0 + out[:, None, :] * a[:, :, None], rdt)
        check_res(to_f32(d), want, rdt, f"hc_combine_rows {rdt}", np.abs(r0) + 2 * np.abs(out)[:, None, :])
        b = torch.full((T, hc, h), float("nan"), device=DEV, dtype=TDT[rdt])
        ops.broadcast_rows(b, to_dev(out))
        assert np.array_equal(to_f32(b), np.broadcast_to(rounded(out, rdt)[:, None, :], (T, hc, h)))
    xn, gate = synth.act(f"t.hc.xn.{h}", T, hc, h), synth.act(f"t.hc.gate.{h}", T, hc, h) * 3
    mixed = torch.empty(T, h, device=DEV)
    ops.hc_mix_rows(to_dev(xn), to_dev(gate), mixed)
    want = orc.hc_mix(xn, gate)
    scale = np.abs(xn).sum(axis=1) / hc
    assert np.all(np.abs(to_f32(mixed) - want) <= 1e-5 * scale + 1e-30), "hc_mix_rows"
    mixed16 = torch.empty(T, h, device=DEV, dtype=torch.bfloat16)
    ops.hc_mix_rows(to_dev(xn, "bf16"), to_dev(gate, "bf16"), mixed16)
    want16 = orc.hc_mix(oracle.round_bf16(xn), oracle.round_bf16(gate))
    assert np.all(np.abs(to_f32(mixed16) - want16) <= 2.0 ** -8 * np.abs(want16) + 1e-5 * scale), "hc_mix_rows bf16"
    y0, x, g = synth.act(f"t.hc.y.{h}", T, h), synth.act(f"t.hc.x.{h}", T, h), synth.act(f"t.hc.g.{h}", T) * 2
    dy = to_dev(y0)
    ops.axpy_sigmoid_rows(dy, to_dev(x), to_dev(g))
    sg = np.array([orc._call("orc_sigmoid", float(v)) for v in g], np.float32)
    wanty = y0 + sg[:, None] * x
    assert np.all(np.abs(to_f32(dy) - wanty) <= 3e-7 * (np.abs(y0) + np.abs(sg[:, None] * x)) + 1e-30), "axpy_sigmoid_rows"


def test_hc_rejects_bad_arguments():
    res = torch.zeros(2, 4, 64, device=DEV)
    out, inj, w = torch.zeros(2, 64, device=DEV), torch.zeros(2, 4, device=DEV), torch.ones(4, 64, device=DEV)
    with pytest.raises(HaloError, match="inject goes with"):
        ops.hc_combine_norm(res, out, None, w, EPS, y=torch.empty_like(res))
    with pytest.raises(HaloError, match="dtype combination"):
        ops.hc_combine_norm(res, out.half(), inj, w, EPS, y=torch.empty_like(res, dtype=torch.bfloat16))
    with pytest.raises(HaloError, match="at most 8"):
        ops.hc_combine_norm(res, out, inj, w, EPS, iw=torch.zeros(9, 256, device=DEV), ipart=torch.zeros(2, 4, 9, device=DEV))
    with pytest.raises(HaloError, match="K-blocked"):
        ops.hc_combine_norm(res[:, :, :40].contiguous(), out[:, :40].contiguous(), inj, w[:, :40].contiguous(), EPS,
                            y16=torch.zeros(2, 4, 40, device=DEV, dtype=torch.float16), y16_tokens=2)
    # empty chunk: a no-op
    ops.hc_combine_norm(torch.empty(0, 4, 64, device=DEV), torch.empty(0, 64, device=DEV), torch.empty(0, 4, device=DEV),
                        w, EPS, y=torch.empty(0, 4, 64, device=DEV))
    torch.cuda.synchronize()


def test_full_size_hc_properties(orc):
    s, T, hc = synth.FULL, 4096, 4
    h = s.hidden
    g = torch.Generator(device=DEV).manual_seed(synth.SEED + 7)
    res = torch.randn(T, hc, h, device=DEV, generator=g).bfloat16()
    out = torch.randn(T, h, device=DEV, generator=g).bfloat16()
    inject = torch.randn(T, hc, device=DEV, generator=g) * 2
    w = to_dev((1 + 0.1 * synth.act("t.hc.full.w", hc, h)).astype(np.float32))
    res0 = res.clone()
    y = torch.empty_like(res)
    ops.hc_combine_norm(res, out, inject, w, EPS, y=y)
    pick = np.unique(synth.rng("t.hc.full.pick").integers(0, T, size=40))
    want_res = to_f32(res0[pick])
    orc.hc_combine_norm(want_res, to_f32(out[pick]), to_f32(inject[pick]), to_f32(w), EPS, 1)
    check_res(to_f32(res[pick]), want_res, "bf16", "full-size residual")
    want_y = orc.hc_combine_norm(to_f32(res[pick]).copy(), None, None, to_f32(w), EPS, 0)
    assert_bf16_within_1ulp(y[pick].view(torch.int16).cpu().numpy().view(np.uint16), want_y, what="full-size grouped norm")
    # every stream of every token has unit mean square before the gamma
    ms = ((y.float() / w) ** 2).mean(dim=2)
    assert float((ms - 1).abs().max()) < 2e-2
    # the separate combine kernel stores the same residual as the fused one
    res2 = res0.clone()
    ops.hc_combine_rows(res2, out, inject)
    assert torch.equal(res2.view(torch.int16), res.view(torch.int16))


# ---- the reference's own launches, by kernel name --------------------------------------------------
@pytest.fixture(scope="module")
def dev():
    return Device.create(0)


def up(dev, a):
    b = dev.alloc(a.nbytes)
    dev.upload(b, 0, a)
    return b


def test_flash_next_combine_sequence_by_name(dev, orc):
    """Broadcast of the embedding into the streams, a combine + grouped norm with inject partials and
    their reduction, the mix, and the token-level MoE form, launched as src/engine/prefill_chunk.cpp:1374-1437
    launches them."""
    T, hc, H, irows, k = 6, 4, 256, 4, 3
    embd = synth.act("t.hcn.embd", T, H)
    out = synth.act("t.hcn.out", T, H)
    inject = synth.act("t.hcn.inj", T, hc)
    w = (1 + 0.1 * synth.act("t.hcn.w", hc, H)).astype(np.float32)
    iw = (synth.act("t.hcn.iw", irows, hc * H) * 0.05).astype(np.float32)
    b_res, b_embd, b_out, b_inj, b_w, b_iw = (dev.alloc(T * hc * H * 4), up(dev, embd), up(dev, out), up(dev, inject),
                                              up(dev, w), up(dev, iw))
    dev.launch(dev.kernel("halo_broadcast_rows"), ((T * hc * H + 255) // 256,), (256,),
               [Arg.Buf(b_res), Arg.Buf(b_embd), Arg.U32(hc), Arg.U32(H), Arg.U32(T)])
    b_xn, b_xh, b_ipart, b_rs = dev.alloc(T * hc * H * 4), dev.alloc(T * hc * H * 2), dev.alloc(T * hc * irows * 4), dev.alloc(T * hc * 4)
    dev.launch(dev.kernel("halo_hc_combine_norm_rows"), (T * hc,), (256,),
               [Arg.Buf(b_res), Arg.Buf(b_out), Arg.Buf(b_inj), Arg.Buf(b_w), Arg.Buf(b_xn), Arg.Buf(b_xh), Arg.U32(hc),
                Arg.U32(H), Arg.F32(EPS), Arg.Buf(b_iw), Arg.Buf(b_ipart), Arg.U32(irows), Arg.U64(0), Arg.U32(0)])
    b_inj2 = dev.alloc(T * irows * 4)
    dev.launch(dev.kernel("halo_inject_reduce"), ((T * irows + 255) // 256,), (256,),
               [Arg.Buf(b_ipart), Arg.Buf(b_inj2), Arg.U32(hc), Arg.U32(irows), Arg.U32(T)])
    want_res = np.broadcast_to(embd[:, None, :], (T, hc, H)).copy()
    orc.hc_combine_norm(want_res, out, inject, w, EPS, 0)
    got_res = dev.download(b_res, 0, T * hc * H * 4, np.float32).reshape(T, hc, H)
    check_res(got_res, want_res, "f32", "by-name residual", np.abs(embd)[:, None, :] + 2 * np.abs(out)[:, None, :])
    want_y = orc.hc_combine_norm(got_res.copy(), None, None, w, EPS, 0)
    got_y = dev.download(b_xn, 0, T * hc * H * 4, np.float32).reshape(T, hc, H)
    assert_rows_close(got_y.reshape(-1, H), want_y.reshape(-1, H), what="by-name grouped norm")
    got_h = dev.download(b_xh, 0, T * hc * H * 2, np.float16).reshape(T, hc, H)
    assert np.array_equal(got_h, got_y.astype(np.float16))
    want_inj = orc.hc_inject(got_y.reshape(T, -1), iw)
    got_inj = dev.download(b_inj2, 0, T * irows * 4, np.float32).reshape(T, irows)
    bound = np.abs(got_y.reshape(T, 1, -1) * iw[None]).sum(axis=2)
    assert np.all(np.abs(got_inj - want_inj) <= 1e-5 * bound)
    # the mix
    gate = synth.act("t.hcn.gate", T, hc, H) * 2
    b_gate, b_mixed = up(dev, gate), dev.alloc(T * H * 4)
    dev.launch(dev.kernel("halo_hc_mix_rows"), ((T * H + 255) // 256,), (256,),
               [Arg.Buf(b_xn), Arg.Buf(b_gate), Arg.Buf(b_mixed), Arg.U32(hc), Arg.U32(H), Arg.U32(T)])
    got_m = dev.download(b_mixed, 0, T * H * 4, np.float32).reshape(T, H)
    want_m = orc.hc_mix(got_y, gate)
    assert np.all(np.abs(got_m - want_m) <= 1e-5 * np.abs(got_y).sum(axis=1) / hc + 1e-30)
    # token-level form with the expert sum, bf16 residual
    yp = synth.act("t.hcn.yp", T * k, H).astype(np.float16)
    pos = synth.rng("t.hcn.pos").permutation(T * k).reshape(T, k).astype(np.uint32)
    mw = synth.rng("t.hcn.mw").random((T, k), dtype=np.float32)
    sx, sg = synth.act("t.hcn.sx", T, H), synth.act("t.hcn.sg", T)
    res16 = oracle.round_bf16(got_res)
    b_r16 = up(dev, oracle.bf16_bits(res16))
    b_yp, b_pos, b_mw, b_sx, b_sg = up(dev, yp), up(dev, pos), up(dev, mw), up(dev, sx), up(dev, sg)
    dev.launch(dev.kernel("halo_hc_combine_norm_tok_moev_rb"), (T,), (256,),
               [Arg.Buf(b_r16), Arg.Buf(b_yp), Arg.Buf(b_pos), Arg.Buf(b_mw), Arg.Buf(b_sx), Arg.Buf(b_sg), Arg.U32(k),
                Arg.Buf(b_inj), Arg.Buf(b_w), Arg.Buf(b_xh), Arg.U32(H), Arg.F32(EPS), Arg.Buf(b_iw), Arg.Buf(b_ipart),
                Arg.U32(irows), Arg.Buf(b_rs), Arg.U32(0)])
    want_out = orc.moe_combine(yp.astype(np.float32), pos, mw, sx, sg)
    want16 = res16.copy()
    orc.hc_combine_norm(want16, want_out, inject, w, EPS, 1)
    got16 = oracle.bf16_to_f32(dev.download(b_r16, 0, T * hc * H * 2, np.uint16)).reshape(T, hc, H)
    check_res(got16, want16, "bf16", "by-name MoE residual")
    # widening the 16-bit residual, and the per-row scales
    b_f32 = dev.alloc(T * hc * H * 4)
    dev.launch(dev.kernel("halo_res_to_f32_rb"), ((T * hc * H + 255) // 256,), (256,),
               [Arg.Buf(b_f32), Arg.Buf(b_r16), Arg.U32(T * hc * H)])
    assert np.array_equal(dev.download(b_f32, 0, T * hc * H * 4, np.float32).reshape(T, hc, H), got16)
    b_sc = dev.alloc(T * hc * 4)
    dev.launch(dev.kernel("halo_hc_norm_scales"), (T * hc,), (256,), [Arg.Buf(b_f32), Arg.Buf(b_sc), Arg.U32(H), Arg.F32(EPS)])
    got_sc = dev.download(b_sc, 0, T * hc * 4, np.float32)
    assert np.allclose(got_sc, 1 / np.sqrt((got16.astype(np.float64) ** 2).mean(axis=2).reshape(-1) + EPS), rtol=2e-6)
    assert np.allclose(dev.download(b_rs, 0, T * hc * 4, np.float32), got_sc, rtol=2e-6)


def test_rmsnorm_rows_h_with_inject_partials(dev, orc):
    """halo_rmsnorm_rows_h with iw: the grouped norm of T x hc rows, fp16 copy and partial products."""
    T, hc, d, irows = 5, 4, 256, 3
    x = synth.act("t.rh.x", T * hc, d)
    w = (1 + 0.1 * synth.act("t.rh.w", hc, d)).astype(np.float32)
    iw = (synth.act("t.rh.iw", irows, hc * d) * 0.05).astype(np.float32)
    b_x, b_w, b_iw = up(dev, x), up(dev, w), up(dev, iw)
    b_y, b_y16, b_ip = dev.alloc(x.nbytes), dev.alloc(x.nbytes // 2), dev.alloc(T * hc * irows * 4)
    dev.launch(dev.kernel("halo_rmsnorm_rows_h"), (T * hc,), (256,),
               [Arg.Buf(b_x), Arg.Buf(b_w), Arg.Buf(b_y), Arg.Buf(b_y16), Arg.U32(d), Arg.F32(EPS), Arg.U32(d), Arg.U32(hc),
                Arg.Buf(b_iw), Arg.Buf(b_ip), Arg.U32(irows), Arg.U32(0)])
    got = dev.download(b_y, 0, x.nbytes, np.float32).reshape(T * hc, d)
    want = orc.rmsnorm_rows(x.copy(), w, EPS, w_stride=d, w_period=hc)
    assert_rows_close(got, want, what="halo_rmsnorm_rows_h + iw")
    assert np.array_equal(dev.download(b_x, 0, x.nbytes, np.float32).reshape(T * hc, d), x), "the input is not written"
    ip = dev.download(b_ip, 0, T * hc * irows * 4, np.float32).reshape(T, hc, irows)
    want_inj = orc.hc_inject(got.reshape(T, -1), iw)
    bound = np.abs(got.reshape(T, 1, -1) * iw[None]).sum(axis=2)
    assert np.all(np.abs(ip.sum(axis=1) - want_inj) <= 1e-5 * bound)


def test_row_copies_and_scale_silu_by_name(dev, orc):
    """halo_copy_at(_h) appending a K row at a position held in device memory (src/engine/qwen35_gpu.cpp's
    cache writes), halo_copy, halo_f16_rows, halo_scale_silu(_h)."""
    n, stride, rows = 512, 512, 6
    src = synth.act("t.cp.src", n)
    params = np.zeros(16, np.uint32)
    params[1] = 4  # kHaloPosition
    b_src, b_par = up(dev, src), up(dev, params)
    cache = np.full((rows, stride), 7.0, np.float32)
    b_cache = up(dev, cache)
    dev.launch(dev.kernel("halo_copy_at"), (2,), (256,), [Arg.Buf(b_cache), Arg.Buf(b_src), Arg.Buf(b_par), Arg.U32(1), Arg.U32(stride), Arg.U32(n)])
    want = cache.copy()
    want[4] = src
    assert np.array_equal(dev.download(b_cache, 0, cache.nbytes, np.float32).reshape(rows, stride), want)
    cache16 = np.full((rows, stride), 7.0, np.float16)
    b_c16 = up(dev, cache16)
    dev.launch(dev.kernel("halo_copy_at_h"), (2,), (256,), [Arg.Buf(b_c16), Arg.Buf(b_src), Arg.Buf(b_par), Arg.U32(1), Arg.U32(stride), Arg.U32(n)])
    want16 = cache16.copy()
    want16[4] = src.astype(np.float16)
    assert np.array_equal(dev.download(b_c16, 0, cache16.nbytes, np.float16).reshape(rows, stride), want16)
    b_dst = dev.alloc(n * 4)
    dev.launch(dev.kernel("halo_copy"), (2,), (256,), [Arg.Buf(b_dst), Arg.Buf(b_src), Arg.U32(n)])
    assert np.array_equal(dev.download(b_dst, 0, n * 4, np.float32), src)
    b_h = dev.alloc(n * 2)
    dev.launch(dev.kernel("halo_f16_rows"), (2,), (256,), [Arg.Buf(b_src), Arg.Buf(b_h), Arg.U32(n)])
    assert np.array_equal(dev.download(b_h, 0, n * 2, np.float16), src.astype(np.float16))
    # silu(x / hc), in place and as an fp16 copy; odd length takes the scalar kernel
    for m in (n, 77):
        x = synth.act("t.cp.x", m) * 4
        wants = np.array([orc._call("orc_silu", float(np.float32(v) * np.float32(0.25))) for v in x], np.float32)
        b_x, b_y = up(dev, x), dev.alloc(m * 2)
        dev.launch(dev.kernel("halo_scale_silu_h"), (1,), (256,), [Arg.Buf(b_x), Arg.Buf(b_y), Arg.F32(0.25), Arg.U32(m)])
        dev.launch(dev.kernel("halo_scale_silu"), (1,), (256,), [Arg.Buf(b_x), Arg.F32(0.25), Arg.U32(m)])
        got = dev.download(b_x, 0, m * 4, np.float32)
        assert np.all(np.abs(got - wants) <= 1e-5 * np.abs(wants) + 1e-30)
        assert ulps16(dev.download(b_y, 0, m * 2, np.float16).astype(np.float32), wants.astype(np.float16).astype(np.float32), "f16").max() <= 1


@pytest.mark.parametrize("T,k,n", [(5, 10, 2048), (3, 10, 2560), (7, 2, 256), (4, 17, 512), (3, 3, 100)])
@pytest.mark.parametrize("ydt,sdt,odt", [("f16", "f32", "f32"), ("f32", "f32", "f32"), ("bf16", "bf16", "bf16"), ("bf16", "f32", "f32")])
def test_moe_combine(orc, T, k, n, ydt, sdt, odt):
    """The routed experts' sum is bit-exact in fp32 (same products and sums in the same order as the CPU
    operator); the gated shared expert adds a term scaled by the device's sigmoid."""
    yp = rounded(synth.act(f"t.moe.yp.{n}", T * k, n), ydt)
    pos = synth.rng(f"t.moe.pos.{n}.{k}").permutation(T * k).reshape(T, k).astype(np.uint32)
    mw = synth.rng(f"t.moe.mw.{n}.{k}").random((T, k), dtype=np.float32)
    sx, sg = rounded(synth.act(f"t.moe.sx.{n}", T, n), sdt), synth.act(f"t.moe.sg.{n}", T)
    d_yp, d_pos, d_mw = to_dev(yp, ydt), torch.from_numpy(pos.view(np.int32)).to(DEV), to_dev(mw)
    out = torch.full((T, n), float("nan"), device=DEV, dtype=TDT[odt])
    ops.moe_combine(d_yp, d_pos, d_mw, out)
    want = orc.moe_combine(yp, pos, mw)
    if odt == "f32":
        assert np.array_equal(to_f32(out), want), "routed sum"
    else:
        assert np.array_equal(oracle.bf16_bits(to_f32(out)), oracle.bf16_bits(want)), "routed sum, bf16 out"
    ops.moe_combine(d_yp, d_pos, d_mw, out, sx=to_dev(sx, sdt), sg=to_dev(sg))
    want2 = orc.moe_combine(yp, pos, mw, sx, sg)
    gs = np.float32(1) / (np.float32(1) + np.exp(-sg, dtype=np.float32))
    mag = np.abs(want) + np.abs(gs[:, None] * sx)
    tol = 3e-7 * mag if odt == "f32" else 2.0 ** -8 * np.abs(want2) + 3e-7 * mag
    assert np.all(np.abs(to_f32(out) - want2) <= tol + 1e-30), "with the shared expert"
    # slots in place (pos None) and the single-slot accumulate of halo_axpy_slot, through the by-name launch
    if ydt == "f32":
        dev = Device.create(0)
        part, w1 = yp[:k], mw[0]
        b_part, b_w, b_out = up(dev, part), up(dev, w1), dev.alloc(n * 4)
        dev.launch(dev.kernel("halo_moe_combine"), (1,), (256,), [Arg.Buf(b_part), Arg.Buf(b_w), Arg.Buf(b_out), Arg.U32(k), Arg.U32(n)])
        acc = np.zeros(n, np.float32)
        for s_ in range(k):
            acc = acc + w1[s_] * part[s_]
        assert np.array_equal(dev.download(b_out, 0, n * 4, np.float32), acc)
        dev.launch(dev.kernel("halo_axpy_slot"), (1,), (256,), [Arg.Buf(b_out), Arg.Buf(b_part), Arg.Buf(b_w), Arg.U32(1), Arg.U32(n)])
        assert np.array_equal(dev.download(b_out, 0, n * 4, np.float32), acc + w1[1] * part[0])
    if ydt == "f16" and n % 8 == 0:
        dev = Device.create(0)
        b_yp, b_pos, b_mw, b_sx, b_sg = up(dev, yp.astype(np.float16)), up(dev, pos), up(dev, mw), up(dev, sx), up(dev, sg)
        b_o = dev.alloc(T * n * 4)
        dev.launch(dev.kernel("halo_moe_combine_grouped"), ((n + 255) // 256, T), (256,),
                   [Arg.Buf(b_yp), Arg.Buf(b_pos), Arg.Buf(b_mw), Arg.Buf(b_o), Arg.U32(k), Arg.U32(n)])
        assert np.array_equal(dev.download(b_o, 0, T * n * 4, np.float32).reshape(T, n), want)
        dev.launch(dev.kernel("halo_moe_combine_shared"), ((n + 255) // 256, T), (256,),
                   [Arg.Buf(b_yp), Arg.Buf(b_pos), Arg.Buf(b_mw), Arg.Buf(b_sx), Arg.Buf(b_sg), Arg.Buf(b_o), Arg.U32(k), Arg.U32(n)])
        assert np.all(np.abs(dev.download(b_o, 0, T * n * 4, np.float32).reshape(T, n) - want2) <= 3e-7 * mag + 1e-30)


def test_committed_outputs_of_the_compiled_reference():
    """The kernels against tests/golden/ops_wide_c1.npz: outputs of the reference's own CPU operators on the
    tiny configuration (generated by tests/golden/make_golden.py where the reference checkout is present)."""
    from conftest import GOLDEN
    g, s = np.load(GOLDEN / "ops_wide_c1.npz"), synth.C1
    T, hc, h = g["hc_res"].shape
    for name, rdt in (("f32", "f32"), ("bf16", "bf16"), ("f16", "f16")):
        d_res = to_dev(rounded(g["hc_res"], rdt), rdt)
        y = torch.empty(T, hc, h, device=DEV)
        ops.hc_combine_norm(d_res, to_dev(g["hc_out"]), to_dev(g["hc_inject"]), to_dev(g["hc_gamma"]), s.eps, y=y)
        check_res(to_f32(d_res), g[f"hc_res_out_{name}"], rdt, f"golden residual {name}",
                  np.abs(g["hc_res"]) + 2 * np.abs(g["hc_out"])[:, None, :])
        if rdt == "f32":  # (16-bit residuals may differ from the fixture by an ulp, so their norms are checked two-stage elsewhere)
            assert_rows_close(to_f32(y).reshape(-1, h), g["hc_y_f32"].reshape(-1, h), rel=2e-5, what="golden grouped norm")
    y32 = to_dev(g["hc_y_f32"])
    irows = g["hc_iw"].shape[0]
    ipart, inj = torch.empty(T, hc, irows, device=DEV), torch.empty(T, irows, device=DEV)
    # norm-only form on rows that are already the fixture's y: unit gammas keep y / rms(y), whose inject
    # partials must add up to the fixture's projection of that y
    yn = torch.empty(T, hc, h, device=DEV)
    ops.hc_combine_norm(y32.clone(), None, None, torch.ones(hc, h, device=DEV), s.eps, y=yn, iw=to_dev(g["hc_iw"]), ipart=ipart)
    ops.inject_reduce(ipart, inj)
    want_inj = np.einsum("tc,rc->tr", to_f32(yn).reshape(T, -1).astype(np.float64), g["hc_iw"].astype(np.float64))
    bound = np.abs(to_f32(yn).reshape(T, 1, -1) * g["hc_iw"][None]).sum(axis=2)
    assert np.all(np.abs(to_f32(inj) - want_inj) <= 1e-5 * bound + 1e-30)
    mixed = torch.empty(T, h, device=DEV)
    ops.hc_mix_rows(y32, to_dev(g["hc_gate"]), mixed)
    assert np.all(np.abs(to_f32(mixed) - g["hc_mixed"]) <= 1e-5 * np.abs(g["hc_y_f32"]).sum(axis=1) / hc + 1e-30)
    out = torch.empty(T, h, device=DEV)
    ops.moe_combine(to_dev(g["moe_yp"], "f16"), torch.from_numpy(g["moe_pos"].view(np.int32)).to(DEV), to_dev(g["moe_w"]), out)
    assert np.array_equal(to_f32(out), g["moe_routed"])
    ops.moe_combine(to_dev(g["moe_yp"], "f16"), torch.from_numpy(g["moe_pos"].view(np.int32)).to(DEV), to_dev(g["moe_w"]), out,
                    sx=to_dev(g["moe_sx"]), sg=to_dev(g["moe_sg"]))
    assert np.all(np.abs(to_f32(out) - g["moe_out"]) <= 3e-7 * (np.abs(g["moe_routed"]) + np.abs(g["moe_sx"])) + 1e-30)
    C = g["conv_x"].shape[1]
    cout, cst = torch.empty(T, C, device=DEV), to_dev(g["conv_state"])
    ops.conv_l2norm(to_dev(g["conv_x"]), cst, to_dev(g["conv_w"]), cout, l2_channels=2 * s.k_heads * s.lin_dim, d=s.lin_dim, eps=s.eps)
    assert_rows_close(to_f32(cout).reshape(-1, s.lin_dim), g["conv_out"].reshape(-1, s.lin_dim), what="golden conv")
    ops.conv_state_advance(to_dev(g["conv_x"]), cst)
    assert np.array_equal(cst.cpu().numpy(), g["conv_state_out"])


@pytest.mark.parametrize("T,hc,h,irows,rdt", [(9, 4, 2048, 4, "bf16"), (6, 4, 2560, 8, "bf16"), (7, 4, 256, 3, "f32"),
                                              (5, 2, 512, 5, "f16"), (3, 4, 8192, 4, "bf16")])
def test_inject_partials_in_a_pass_of_their_own(orc, T, hc, h, irows, rdt):
    """Where the fp32 normalized values can be had again (an fp32 y, or the stored residual and the row scales),
    the partial products run as a second pass with the weights in registers; it must agree with the products
    computed inside the combine kernel, and with the oracle's projection of the fp32 y."""
    res, out, inject, w = inputs(f"t.hc.inj2.{h}", T, hc, h, rdt, "f32")
    iw = (synth.act(f"t.hc.inj2.iw.{h}", irows, hc * h) * 0.05).astype(np.float32)

    def run(fused, with_y32, with_rscale):
        lib().tune("hc_fused_inject", fused)
        try:
            d_res = to_dev(res, rdt)
            y = torch.empty(T, hc, h, device=DEV) if with_y32 else None
            y16 = torch.empty(T, hc, h, device=DEV, dtype=torch.float16)
            rscale = torch.empty(T, hc, device=DEV) if with_rscale else None
            ipart = torch.full((T, hc, irows), float("nan"), device=DEV)
            ops.hc_combine_norm(d_res, to_dev(out), to_dev(inject), to_dev(w), EPS, y=y, y16=y16, rscale=rscale,
                                iw=to_dev(iw), ipart=ipart)
            return to_f32(ipart), (to_f32(y) if with_y32 else None), to_f32(d_res)
        finally:
            lib().tune("hc_fused_inject", 0)

    fused, y32, res_after = run(1, True, True)
    want = orc.hc_inject(y32.reshape(T, -1), iw)
    bound = np.abs(y32.reshape(T, hc, 1, h) * iw.reshape(1, irows, hc, h).transpose(0, 2, 1, 3)).sum(axis=3)  # [T, hc, irows]
    tot = bound.sum(axis=1)
    assert np.all(np.abs(fused.sum(axis=1) - want) <= 1e-5 * tot + 1e-30), "in-kernel products"
    for with_y32, with_rscale in ((False, True), (True, False), (True, True)):  # rebuild from res, fp32 y, rebuild preferred
        got, _, res2 = run(0, with_y32, with_rscale)
        assert np.array_equal(res2, res_after)
        assert np.all(np.abs(got - fused) <= 2e-6 * bound + 1e-30), f"second pass (y32={with_y32}, rscale={with_rscale}) vs in-kernel"
        assert np.all(np.abs(got.sum(axis=1) - want) <= 1e-5 * tot + 1e-30)
