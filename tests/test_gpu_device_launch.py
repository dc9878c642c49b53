"""The reference-shaped host path (GPU only): kernels looked up by name and launched with the
reference's own grid, block and ordered argument list through the Device mirror of
rt::Device, written the way the reference's kernel tests are (tests/gpu/quant_gpu_test.cpp):
LCG-seeded uniform inputs, upload, launch by name, download, compare with the CPU operator.
"""
import numpy as np
import pytest

import oracle
from conftest import assert_rows_close
from halo_flash_b200 import HaloError, synth
from halo_flash_b200.device import Arg, Device

pytestmark = pytest.mark.gpu


def lcg_vec(seed, n, amp):
    """The reference tests' input generator (tests/gpu/quant_gpu_test.cpp:2373-2377)."""
    out = np.empty(n, np.float32)
    s = np.uint32(seed)
    with np.errstate(over="ignore"):
        for i in range(n):
            s = np.uint32(s * np.uint32(1664525) + np.uint32(1013904223))
            out[i] = np.float32(amp) * (np.float32(s >> np.uint32(8)) / np.float32(16777216.0) - np.float32(0.5))
    return out, int(s)


@pytest.fixture(scope="module")
def dev():
    return Device.create(0)


def up(dev, a):
    b = dev.alloc(a.nbytes)
    dev.upload(b, 0, a)
    return b


def test_unknown_kernel_is_refused(dev):
    with pytest.raises(HaloError, match="not part"):
        dev.kernel("halo_attention_decode")


def test_rmsnorm_rows_and_l2norm_by_name(dev, orc):
    T, hc, d = 6, 4, 320
    x, seed = lcg_vec(7, T * hc * d, 6.0)
    w, _ = lcg_vec(seed, hc * d, 2.0)
    bx, bw, by = up(dev, x), up(dev, w), dev.alloc(x.nbytes)
    dev.launch(dev.kernel("halo_rmsnorm_rows"), (T * hc,), (256,),
               [Arg.Buf(bx), Arg.Buf(bw), Arg.Buf(by), Arg.U32(d), Arg.F32(1e-6), Arg.U32(d), Arg.U32(hc)])
    got = dev.download(by, 0, x.nbytes, np.float32).reshape(T * hc, d)
    want = orc.rmsnorm_rows(x.reshape(T * hc, d).copy(), w.reshape(hc, d), 1e-6, w_stride=d, w_period=hc)
    assert_rows_close(got, want, what="halo_rmsnorm_rows")
    # byte offsets into a scratch arena, as the engine slices its buffers
    arena = dev.alloc(x.nbytes + 4096)
    dev.upload(arena, 4096, x)
    dev.launch(dev.kernel("halo_l2norm"), (T * hc,), (128,), [Arg.Buf(arena, 4096), Arg.U32(d), Arg.F32(1e-6)])
    got = dev.download(arena, 4096, x.nbytes, np.float32).reshape(T * hc, d)
    assert_rows_close(got, orc.l2norm_rows(x.reshape(T * hc, d).copy(), 1e-6), what="halo_l2norm")


def test_qwen35_layer_sequence_by_name(dev, orc):
    """The elementwise calls of Qwen35Gpu::PrefillChunk for one GQA layer, in the engine's order and
    with its launch shapes (src/engine/qwen35_gpu.cpp:469-574): rmsnorm, split_qgate, per-head
    rmsnorm of q and k, rope_neox_rows twice, add, rmsnorm, silu_mul, add."""
    s, T = synth.C1, 5
    H, nh, nkv, hd = s.hidden, s.q_heads, s.kv_heads, s.head_dim
    res, seed = lcg_vec(11, T * H, 4.0)
    g_attn, seed = lcg_vec(seed, H, 1.0)
    g_attn += 1
    qg, seed = lcg_vec(seed, T * nh * 2 * hd, 3.0)
    kk, seed = lcg_vec(seed, T * nkv * hd, 3.0)
    gq, seed = lcg_vec(seed, hd, 1.0)
    gq += 1
    attn_out, seed = lcg_vec(seed, T * H, 2.0)
    gate, seed = lcg_vec(seed, T * s.ff, 5.0)
    upv, seed = lcg_vec(seed, T * s.ff, 5.0)
    pos0 = 1000
    b = {k: up(dev, v) for k, v in dict(res=res, g=g_attn, qg=qg, k=kk, gq=gq, ao=attn_out, gate=gate, up=upv).items()}
    xn, q, gt = dev.alloc(res.nbytes), dev.alloc(T * nh * hd * 4), dev.alloc(T * nh * hd * 4)
    K = dev.kernel
    dev.launch(K("halo_rmsnorm"), (T,), (256,), [Arg.Buf(b["res"]), Arg.Buf(b["g"]), Arg.Buf(xn), Arg.U32(H),
                                                Arg.F32(s.eps), Arg.U32(0)])
    dev.launch(K("halo_split_qgate"), (T * nh,), (256,), [Arg.Buf(b["qg"]), Arg.Buf(q), Arg.Buf(gt), Arg.U32(hd)])
    dev.launch(K("halo_rmsnorm"), (T * nh,), (256,), [Arg.Buf(q), Arg.Buf(b["gq"]), Arg.Buf(q), Arg.U32(hd),
                                                     Arg.F32(s.eps), Arg.U32(0)])
    dev.launch(K("halo_rmsnorm"), (T * nkv,), (256,), [Arg.Buf(b["k"]), Arg.Buf(b["gq"]), Arg.Buf(b["k"]), Arg.U32(hd),
                                                      Arg.F32(s.eps), Arg.U32(0)])
    dev.launch(K("halo_rope_neox_rows"), (T * nh,), (64,), [Arg.Buf(q), Arg.U32(hd), Arg.U32(s.rot), Arg.U32(pos0),
                                                           Arg.U32(nh), Arg.F32(s.theta)])
    dev.launch(K("halo_rope_neox_rows"), (T * nkv,), (64,), [Arg.Buf(b["k"]), Arg.U32(hd), Arg.U32(s.rot),
                                                            Arg.U32(pos0), Arg.U32(nkv), Arg.F32(s.theta)])
    dev.launch(K("halo_add"), ((T * H + 255) // 256,), (256,), [Arg.Buf(b["res"]), Arg.Buf(b["ao"]), Arg.U32(T * H)])
    dev.launch(K("halo_silu_mul"), ((T * s.ff + 255) // 256,), (256,), [Arg.Buf(b["gate"]), Arg.Buf(b["up"]),
                                                                       Arg.U32(T * s.ff)])
    dev.synchronize()
    pos = np.arange(pos0, pos0 + T, dtype=np.uint32)
    assert_rows_close(dev.download(xn, 0, res.nbytes, np.float32).reshape(T, H),
                      orc.rmsnorm_rows(res.reshape(T, H).copy(), g_attn, s.eps), what="attn_norm")
    qsplit = np.ascontiguousarray(qg.reshape(T * nh, 2, hd)[:, 0])
    wq = orc.rope_rows(orc.rmsnorm_rows(qsplit.copy(), gq, s.eps).reshape(T, nh, hd), pos, s.rot, s.theta)
    assert_rows_close(dev.download(q, 0, T * nh * hd * 4, np.float32).reshape(-1, hd), wq.reshape(-1, hd), what="q")
    wk = orc.rope_rows(orc.rmsnorm_rows(kk.reshape(T * nkv, hd).copy(), gq, s.eps).reshape(T, nkv, hd), pos, s.rot,
                       s.theta)
    assert_rows_close(dev.download(b["k"], 0, kk.nbytes, np.float32).reshape(-1, hd), wk.reshape(-1, hd), what="k")
    assert dev.download(gt, 0, T * nh * hd * 4, np.float32).tobytes() == \
        np.ascontiguousarray(qg.reshape(T * nh, 2, hd)[:, 1]).tobytes()
    assert dev.download(b["res"], 0, res.nbytes, np.float32).tobytes() == (res + attn_out).tobytes()
    got = dev.download(b["gate"], 0, gate.nbytes, np.float32).astype(np.float64)
    want = orc.silu_mul(gate.copy(), upv)
    assert np.all(np.abs(got - want) <= 1e-5 * np.abs(want) + 1e-30)


def test_null_optional_pointer_and_cache_append(dev, orc):
    """A null optional pointer travels as Arg::Val<uint64_t>(0) (src/engine/prefill_chunk.cpp:707)."""
    s, T = synth.FULL, 3
    hd, nkv = s.head_dim, s.kv_heads
    x, seed = lcg_vec(5, T * nkv * hd, 4.0)
    w, _ = lcg_vec(seed, hd, 1.0)
    w += 1
    want = orc.rope_rows(orc.rmsnorm_rows(x.reshape(-1, hd).copy(), w, s.eps).reshape(T, nkv, hd),
                         np.arange(70, 70 + T, dtype=np.uint32), s.rot, s.theta).reshape(-1, hd)
    for with_cache in (False, True):
        bx, bw, cache = up(dev, x), up(dev, w), dev.alloc(x.nbytes)
        dev.fill(cache, 0)
        dev.launch(dev.kernel("halo_norm_rope_rows"), (T * nkv,), (256,),
                   [Arg.Buf(bx), Arg.Buf(bw), Arg.F32(s.eps), Arg.U32(hd), Arg.U32(s.rot), Arg.U32(70), Arg.U32(nkv),
                    Arg.F32(s.theta), Arg.Buf(cache) if with_cache else Arg.Null])
        got = dev.download(bx, 0, x.nbytes, np.float32).reshape(-1, hd)
        assert_rows_close(got, want, what="norm_rope_rows")
        c = dev.download(cache, 0, x.nbytes, np.float32).reshape(-1, hd)
        assert c.tobytes() == (got.tobytes() if with_cache else np.zeros_like(got).tobytes())


def test_captured_graph_replays_with_device_resident_step_values(dev, orc):
    """Per-step values live in device memory so one recorded graph replays at any token and
    position (src/kernels/step_params.h:4-15; src/rt/device.hpp:66-75): embed_p + rope_neox_p."""
    s = synth.C1
    table = synth.q8_0_table("t.g.table", 256, s.hidden)
    x, _ = lcg_vec(3, s.q_heads * s.head_dim, 2.0)
    btab, params = up(dev, table), dev.alloc(64)
    out, bx = dev.alloc(s.hidden * 4), dev.alloc(x.nbytes)
    dev.upload(params, 0, np.array([0] * 16, np.uint32))
    dev.begin_capture()
    with pytest.raises(HaloError):
        dev.synchronize()
    dev.launch(dev.kernel("halo_matvec_q8_0_embed_p"), ((s.hidden + 255) // 256,), (256,),
               [Arg.Buf(btab), Arg.Buf(out), Arg.Buf(params), Arg.U32(s.hidden), Arg.U64(s.q8_row_bytes)])
    dev.launch(dev.kernel("halo_rope_neox_p"), (s.q_heads,), (64,),
               [Arg.Buf(bx), Arg.Buf(params), Arg.U32(s.head_dim), Arg.U32(s.rot), Arg.U32(1), Arg.U32(1),
                Arg.F32(s.theta)])
    graph = dev.end_capture()
    for token, pos in ((17, 0), (255, 4095), (3, 123)):
        step = np.zeros(16, np.uint32)
        step[0], step[1] = token, pos
        dev.upload(params, 0, step)
        dev.upload(bx, 0, x)
        dev.launch_graph(graph)
        dev.synchronize()
        assert dev.download(out, 0, s.hidden * 4, np.float32).tobytes() == \
            orc.embed_q8_0_rows(table, np.array([token], np.uint32), s.hidden).tobytes()
        got = dev.download(bx, 0, x.nbytes, np.float32).reshape(1, s.q_heads, s.head_dim)
        want = orc.rope_rows(x.reshape(1, s.q_heads, s.head_dim).copy(), np.array([pos], np.uint32), s.rot, s.theta)
        assert np.all(np.abs(got - want) <= 1e-5 * np.maximum(np.abs(x).max(), 1e-30))
    dev.free_graph(graph)
