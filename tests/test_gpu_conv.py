"""Parity of the Gated DeltaNet conv + SiLU + L2 norm kernels with the CPU oracle (GPU only).

The oracle repeats the conv loop of Qwen35Reference::Linear (src/model/qwen35.cpp:180-198) around the
reference's cpu::Silu and cpu::L2Norm. Tolerances: fp32 outputs within 1e-5 of max(|want|, rms(head));
16-bit outputs within 1 ulp of the rounded oracle value (2 where the conv sum cancels); the conv state
after a chunk bit-exact (it is a copy of inputs). A chunk run in pieces (state advanced in between) equals
the chunk run at once bit for bit, the property the reference's prefill kernels are built to keep
(src/kernels/core.hip:3480-3484).
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import assert_rows_close
from halo_flash_b200 import HaloError, lib, ops, synth
from halo_flash_b200.device import Arg, Device

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
EPS = 1e-6
TDT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


def to_dev(a, dtype="f32"):
    if dtype == "bf16":
        return torch.from_numpy(oracle.bf16_bits(a).view(np.int16)).to(DEV).view(torch.bfloat16).reshape(a.shape)
    if dtype == "f16":
        return torch.from_numpy(a.astype(np.float16)).to(DEV)
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def rounded(a, dtype):
    if dtype == "bf16":
        return oracle.round_bf16(a)
    if dtype == "f16":
        return a.astype(np.float16).astype(np.float32)
    return a


def make(tag, T, C, kern):
    x = synth.act(tag + ".x", T, C)
    state = synth.act(tag + ".s", max(kern - 1, 1), C)[:kern - 1]
    w = (synth.act(tag + ".w", C, kern) * 0.5).astype(np.float32)
    return x, np.ascontiguousarray(state), w


def check(got, want, d, odt, what):
    heads = want.reshape(-1, d)
    if odt == "f32":
        assert_rows_close(got.reshape(-1, d), heads, what=what)
    else:
        eps16 = 2.0 ** -8 if odt == "bf16" else 2.0 ** -11
        rms = np.sqrt((heads.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
        tol = eps16 * np.abs(heads) + 1e-5 * np.maximum(np.abs(heads), rms)
        assert np.all(np.abs(got.reshape(-1, d) - heads) <= tol + 1e-30), what


@pytest.mark.parametrize("T,C,l2,d,kern", [(1, 512, 256, 64, 4), (7, 512, 256, 64, 4), (8, 512, 256, 64, 4),
                                           (29, 8192, 4096, 128, 4), (5, 384, 256, 128, 4), (6, 512, 0, 128, 4),
                                           (9, 200, 100, 50, 4), (6, 256, 128, 64, 3), (4, 256, 128, 64, 2), (3, 128, 64, 64, 1)])
@pytest.mark.parametrize("idt,odt", [("f32", "f32"), ("f16", "f32"), ("f16", "f16"), ("bf16", "bf16"), ("bf16", "f32")])
@pytest.mark.parametrize("staged", [1, 0])
def test_conv_l2norm(orc, T, C, l2, d, kern, idt, odt, staged):
    """staged: rows brought into shared memory by bulk asynchronous copies (the default), or held in registers."""
    x, state, w = make(f"t.conv.{T}.{C}.{kern}", T, C, kern)
    x = rounded(x, idt)
    out = torch.full((T, C), float("nan"), device=DEV, dtype=TDT[odt])
    d_state = to_dev(state) if kern > 1 else None
    lib().tune("conv_staged", staged)
    try:
        ops.conv_l2norm(to_dev(x, idt), d_state, to_dev(w), out, l2_channels=l2, d=d, eps=EPS)
    finally:
        lib().tune("conv_staged", 1)
    st = state.copy()
    want = orc.conv_l2norm(x, st, w, l2, d, EPS)
    check(out.float().cpu().numpy(), want, d if l2 else C, odt, "conv + SiLU + L2")
    if kern > 1:
        assert torch.equal(d_state, to_dev(state)), "the conv does not write the state"
        ops.conv_state_advance(to_dev(x, idt), d_state)
        assert np.array_equal(d_state.cpu().numpy(), st), "state after the chunk"


def test_chunk_in_pieces_equals_chunk_at_once(orc):
    T, C, l2, d, kern = 37, 1024, 512, 128, 4
    x, state, w = make("t.conv.pieces", T, C, kern)
    dx, dw = to_dev(x, "bf16"), to_dev(w)
    whole = torch.empty(T, C, device=DEV, dtype=torch.bfloat16)
    ops.conv_l2norm(dx, to_dev(state), dw, whole, l2_channels=l2, d=d, eps=EPS)
    st = to_dev(state)
    parts = []
    for b, e in ((0, 1), (1, 3), (3, 12), (12, 13), (13, 37)):  # one token (a decode step), short and long pieces
        piece = torch.empty(e - b, C, device=DEV, dtype=torch.bfloat16)
        chunk = dx[b:e].contiguous()
        ops.conv_l2norm(chunk, st, dw, piece, l2_channels=l2, d=d, eps=EPS)
        ops.conv_state_advance(chunk, st)
        parts.append(piece)
    assert torch.equal(torch.cat(parts).view(torch.int16), whole.view(torch.int16))
    assert np.array_equal(st.cpu().numpy(), oracle.round_bf16(x)[-3:])
    # the register form of the kernel computes the same bits as the staged form
    lib().tune("conv_staged", 0)
    try:
        regs = torch.empty(T, C, device=DEV, dtype=torch.bfloat16)
        ops.conv_l2norm(dx, to_dev(state), dw, regs, l2_channels=l2, d=d, eps=EPS)
    finally:
        lib().tune("conv_staged", 1)
    assert torch.equal(regs.view(torch.int16), whole.view(torch.int16))


def test_no_staging_wait_ever_ran_out():
    """The staged kernel's barrier wait is bounded; a wait that runs out is counted. After the tests above: zero."""
    import ctypes as C
    n = C.c_uint(123)
    err = C.create_string_buffer(256)
    f = lib().cdll.halo_b200_conv_stage_timeouts
    f.restype, f.argtypes = C.c_int, [C.POINTER(C.c_uint), C.c_char_p, C.c_size_t]
    assert f(C.byref(n), err, len(err)) == 0, err.value
    assert n.value == 0


def test_conv_rejects_bad_arguments():
    x = torch.zeros(4, 256, device=DEV)
    w, st = torch.zeros(256, 4, device=DEV), torch.zeros(3, 256, device=DEV)
    with pytest.raises(HaloError, match="must not be the same buffer"):
        ops.conv_l2norm(x, st, w, x, l2_channels=128, d=64, eps=EPS)
    with pytest.raises(HaloError, match="whole heads"):
        ops.conv_l2norm(x, st, w, torch.empty_like(x), l2_channels=100, d=64, eps=EPS)
    with pytest.raises(HaloError, match="dtype pair"):
        ops.conv_l2norm(x, st, w, torch.empty(4, 256, device=DEV, dtype=torch.bfloat16), l2_channels=128, d=64, eps=EPS)
    ops.conv_l2norm(x[:0], st, w, torch.empty(0, 256, device=DEV), l2_channels=128, d=64, eps=EPS)  # empty chunk
    torch.cuda.synchronize()


def test_full_size_conv_properties(orc):
    """Config-4 shape: 8192 conv channels (q, k: 2 x 16 heads x 128, normalized; v: 32 x 128), T = 4096, bf16."""
    s, T = synth.FULL, 4096
    C, l2, d = 2 * s.k_heads * s.lin_dim + s.v_heads * s.lin_dim, 2 * s.k_heads * s.lin_dim, s.lin_dim
    g = torch.Generator(device=DEV).manual_seed(synth.SEED + 11)
    x = torch.randn(T, C, device=DEV, generator=g).bfloat16()
    w = torch.randn(C, 4, device=DEV, generator=g) * 0.5
    st = torch.randn(3, C, device=DEV, generator=g)
    out = torch.empty_like(x)
    ops.conv_l2norm(x, st, w, out, l2_channels=l2, d=d, eps=EPS)
    # q / k heads have unit length (up to bf16 rounding)
    n = (out[:, :l2].float().view(T, -1, d) ** 2).sum(dim=2)
    assert float((n - 1).abs().max()) < 2e-2
    # sampled windows against the oracle: tokens b-3 .. b+5 with the true history as the state
    for b in (0, 5, 1234, 4090):
        e = min(T, b + 6)
        hist = np.zeros((3, C), np.float32)
        for j in range(3):
            i = b - 3 + j
            hist[j] = x[i].float().cpu().numpy() if i >= 0 else st[i + 3].cpu().numpy()
        want = orc.conv_l2norm(x[b:e].float().cpu().numpy(), hist, w.cpu().numpy(), l2, d, EPS)
        check(out[b:e].float().cpu().numpy(), want, d, "bf16", f"full-size conv rows {b}..{e}")


def test_conv_kernels_by_name(orc):
    """The engine's launches (src/engine/qwen35_gpu.cpp:487-493, src/engine/prefill_chunk.cpp:555-601,
    src/engine/flash_next_gpu.cpp:523, 555): prefill8 + state advance, then decode steps."""
    dev = Device.create(0)
    T, C, l2, d, kern = 13, 1024, 512, 128, 4
    x, state, w = make("t.conv.name", T + 2, C, kern)

    def up(a):
        b = dev.alloc(a.nbytes)
        dev.upload(b, 0, a)
        return b

    b_x, b_st, b_w, b_out = up(x[:T]), up(state), up(w), dev.alloc(T * C * 4)
    dev.launch(dev.kernel("halo_conv_l2norm_prefill8"), (C // 128, (T + 7) // 8), (128,),
               [Arg.Buf(b_x), Arg.Buf(b_st), Arg.Buf(b_w), Arg.Buf(b_out), Arg.U32(C), Arg.U32(T), Arg.U32(l2), Arg.F32(EPS)])
    dev.launch(dev.kernel("halo_conv_state_advance"), ((C + 255) // 256,), (256,),
               [Arg.Buf(b_x), Arg.Buf(b_st), Arg.U32(C), Arg.U32(kern), Arg.U32(T)])
    st = state.copy()
    want = orc.conv_l2norm(x[:T], st, w, l2, d, EPS)
    got = dev.download(b_out, 0, T * C * 4, np.float32).reshape(T, C)
    check(got, want, d, "f32", "halo_conv_l2norm_prefill8")
    assert np.array_equal(dev.download(b_st, 0, 3 * C * 4, np.float32).reshape(3, C), st)
    # the one-token prefill form gives the same bits as the tiled one
    b_out1 = dev.alloc(T * C * 4)
    b_st0 = up(state)
    dev.launch(dev.kernel("halo_conv_l2norm_prefill"), (C // 128, T), (128,),
               [Arg.Buf(b_x), Arg.Buf(b_st0), Arg.Buf(b_w), Arg.Buf(b_out1), Arg.U32(C), Arg.U32(kern), Arg.U32(l2), Arg.F32(EPS)])
    assert np.array_equal(dev.download(b_out1, 0, T * C * 4, np.float32).reshape(T, C), got)
    # two decode steps: the state moves with each
    for t in (T, T + 1):
        b_in, b_o = up(x[t]), dev.alloc(C * 4)
        dev.launch(dev.kernel("halo_conv_l2norm"), (C // 128,), (128,),
                   [Arg.Buf(b_in), Arg.Buf(b_st), Arg.Buf(b_w), Arg.Buf(b_o), Arg.U32(C), Arg.U32(kern), Arg.U32(l2), Arg.F32(EPS)])
        want1 = orc.conv_l2norm(x[t:t + 1], st, w, l2, d, EPS)
        check(dev.download(b_o, 0, C * 4, np.float32).reshape(1, C), want1, d, "f32", "halo_conv_l2norm step")
        assert np.array_equal(dev.download(b_st, 0, 3 * C * 4, np.float32).reshape(3, C), st)
    # halo_conv_step: no normalization
    b_in, b_o = up(x[0]), dev.alloc(C * 4)
    dev.launch(dev.kernel("halo_conv_step"), ((C + 255) // 256,), (256,),
               [Arg.Buf(b_in), Arg.Buf(b_st), Arg.Buf(b_w), Arg.Buf(b_o), Arg.U32(C), Arg.U32(kern)])
    want2 = orc.conv_l2norm(x[0:1], st, w, 0, d, EPS)
    check(dev.download(b_o, 0, C * 4, np.float32).reshape(1, C), want2, C, "f32", "halo_conv_step")


@pytest.mark.parametrize("B,C,l2,d,kern", [(1, 512, 256, 128, 4), (3, 1024, 512, 128, 4), (4, 320, 128, 64, 3),
                                           (2, 200, 0, 128, 2), (2, 256, 256, 128, 1)])
def test_conv_step_entries(orc, B, C, l2, d, kern):
    """halo_conv_l2norm_y (src/kernels/batch_decode.hip:1741-1748): one launch steps B sessions, each with its own
    conv state found through a table of device addresses; every entry equals the single-session step bit for bit
    and the oracle within tolerance, and each state moves by its entry's input."""
    st = torch.cuda.current_stream().cuda_stream
    x, _, w = make("t.conv.y", B, C, kern)
    stride = C + 24  # entries are slices of a wider scratch row
    xin = np.zeros((B, stride), np.float32)
    xin[:, :C] = x
    states = [np.ascontiguousarray(synth.act(f"t.conv.y.s{e}", max(kern - 1, 1), C)[:kern - 1]) for e in range(B)]
    d_states = [to_dev(s.copy()) if kern > 1 else torch.zeros(1, device=DEV) for s in states]
    tstride, tslot = 5, 3
    tab = np.zeros((B, tstride), np.uint64)
    for e in range(B):
        tab[e, tslot] = d_states[e].data_ptr()
    d_tab = torch.from_numpy(tab.view(np.int64)).to(DEV)
    d_in, d_w = to_dev(xin), to_dev(w)
    d_out = torch.full((B, stride), 7.0, device=DEV)
    lib().call("conv_l2norm_y", st, d_in.data_ptr(), d_tab.data_ptr(), tstride, tslot, d_w.data_ptr(), d_out.data_ptr(),
               C, kern, l2, EPS, stride, d, B)
    got = d_out.cpu().numpy()
    assert np.all(got[:, C:] == 7.0), "wrote past an entry's channels"
    for e in range(B):
        hist = states[e].copy()
        want = orc.conv_l2norm(x[e:e + 1], hist, w, l2, d, EPS)  # advances hist
        if l2:
            check(got[e:e + 1, :l2], want[:, :l2], d, "f32", f"entry {e} q/k")
        if l2 < C:
            assert_rows_close(got[e:e + 1, l2:C], want[:, l2:], what=f"entry {e} v")
        if kern > 1:
            assert np.array_equal(d_states[e].cpu().numpy(), hist), f"entry {e} state"
        # the single-session step on the same inputs: same bits
        s1 = to_dev(states[e].copy()) if kern > 1 else torch.zeros(1, device=DEV)
        o1 = torch.empty(C, device=DEV)
        lib().call("conv_l2norm", st, d_in[e].data_ptr(), s1.data_ptr(), d_w.data_ptr(), o1.data_ptr(), C, kern, l2, EPS, d)
        assert np.array_equal(o1.cpu().numpy(), got[e, :C])
        # and in place (a thread reads its input before it writes its output)
        s2 = to_dev(states[e].copy()) if kern > 1 else torch.zeros(1, device=DEV)
        io = d_in[e, :C].clone()
        lib().call("conv_l2norm", st, io.data_ptr(), s2.data_ptr(), d_w.data_ptr(), io.data_ptr(), C, kern, l2, EPS, d)
        assert np.array_equal(io.cpu().numpy(), got[e, :C])
    with pytest.raises(HaloError, match="state table"):
        lib().call("conv_l2norm_y", st, d_in.data_ptr(), 0, tstride, tslot, d_w.data_ptr(), d_out.data_ptr(),
                   C, kern, l2, EPS, stride, d, B)
    # no entries: nothing runs
    lib().call("conv_l2norm_y", st, d_in.data_ptr(), 0, tstride, tslot, d_w.data_ptr(), d_out.data_ptr(),
               C, kern, l2, EPS, stride, d, 0)


def test_conv_step_entries_by_name(orc):
    """The batched decoder's launch (grid (channels / 128, B), block 128) through the launch-by-name boundary."""
    dev = Device.create(0)
    B, C, l2, d, kern = 3, 512, 256, 128, 4
    x, _, w = make("t.conv.yn", B, C, kern)

    def up(a):
        b = dev.alloc(a.nbytes)
        dev.upload(b, 0, a)
        return b

    states = [np.ascontiguousarray(synth.act(f"t.conv.yn.s{e}", 3, C)) for e in range(B)]
    d_states = [to_dev(s.copy()) for s in states]
    tab = np.array([[0, s.data_ptr()] for s in d_states], np.uint64)
    b_in, b_tab, b_w, b_out = up(x), up(tab), up(w), dev.alloc(B * C * 4)
    dev.launch(dev.kernel("halo_conv_l2norm_y"), (C // 128, B), (128,),
               [Arg.Buf(b_in), Arg.Buf(b_tab), Arg.U32(2), Arg.U32(1), Arg.Buf(b_w), Arg.Buf(b_out), Arg.U32(C),
                Arg.U32(kern), Arg.U32(l2), Arg.F32(EPS), Arg.U32(C)])
    got = dev.download(b_out, 0, B * C * 4, np.float32).reshape(B, C)
    for e in range(B):
        hist = states[e].copy()
        want = orc.conv_l2norm(x[e:e + 1], hist, w, l2, d, EPS)
        check(got[e:e + 1, :l2], want[:, :l2], d, "f32", f"entry {e}")
        assert_rows_close(got[e:e + 1, l2:], want[:, l2:], what=f"entry {e} v")
        assert np.array_equal(d_states[e].cpu().numpy(), hist)
