"""Generates the committed golden fixtures. Run in a container that has the
reference checkout ($HALO_REFERENCE_ROOT, else a directory named `reference` beside this repository):

    python tests/golden/make_golden.py

1. quant_blocks.tsv - the Q8_0, F16 and BF16 rows of the reference's own golden
   file tests/core/data/quant.tsv (blocks decoded by llama.cpp's gguf-py; format
   `type \t block hex \t fp32 values hex`, tests/core/quant_test.cpp:153-185).
   Data only; the formats outside this path are dropped.
2. ops_c1.npz - inputs and outputs of the reference's OWN CPU operators
   (oracle/_ref/libhalo_ref.so = src/model/cpu_ops.cpp, src/core/quant.cpp,
   src/core/lowbit.cpp compiled unmodified) on the tiny configuration:
   hidden 256, 4 Q / 2 KV heads x 64, rot 16, theta 1e7, 4 value heads x 64,
   ff 128, vocab 4096 Q8_0, T = 32, fp32.
3. ops_wide_c1.npz - the same for the ops around the five groups, on the tiny configuration with 4 residual
   streams: hyper-connection combine + grouped norm, inject projection, mix, the experts' combine, and the
   DeltaNet conv + SiLU + L2 norm. These CPU operators are members of model classes in the reference
   (src/model/reference.cpp:151-202, 558-578; src/model/qwen35.cpp:180-198), so oracle/ref_shim.cpp repeats
   their loops around the reference's own cpu::RmsNorm / L2Norm / Sigmoid / Silu / MatVec.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from halo_flash_b200 import synth  # noqa: E402

HERE = Path(__file__).resolve().parent
T = 32


def extract_quant_blocks() -> int:
    src = oracle.REFERENCE_ROOT / "tests" / "core" / "data" / "quant.tsv"
    keep = [l for l in src.read_text().splitlines() if l.split("\t", 1)[0] in ("Q8_0", "F16", "BF16")]
    (HERE / "quant_blocks.tsv").write_text("\n".join(keep) + "\n")
    return len(keep)


def make_ops() -> dict:
    oracle.build(ref=True)
    ref = oracle.load("reference")
    assert ref.kind == "reference"
    s = synth.C1
    out: dict[str, np.ndarray] = {}
    # group 1: residual add + RMSNorm(1 + w), then Q8_0 of the normalized rows
    res, delta = synth.act("g.res", T, s.hidden), synth.act("g.delta", T, s.hidden)
    w = synth.norm_w("g.norm_w", s.hidden)
    out.update(res=res, delta=delta, norm_w=w)
    summed = res + delta  # one fp32 add per element (src/model/qwen35.cpp:322)
    xn = ref.rmsnorm_rows(summed.copy(), np.float32(1.0) + w, s.eps)
    out.update(res_out=summed, xn=xn, xn_q8_0=ref.encode_q8_0_rows(xn))
    # group 2: q/k L2 norm and the gated RMSNorm
    qk = synth.act("g.qk", T, 2 * s.k_heads, s.lin_dim)
    out.update(qk=qk, qk_l2=ref.l2norm_rows(qk.copy(), s.eps))
    o, z = synth.act("g.o", T, s.v_heads, s.lin_dim), synth.act("g.z", T, s.v_heads, s.lin_dim)
    gw = synth.gated_w("g.gated_w", s.lin_dim)
    out.update(o=o, z=z, gated_w=gw, gated_silu=ref.gated_norm_rows(o.copy(), gw, z, s.eps, mode=0),
               gated_sigmoid=ref.gated_norm_rows(o.copy(), gw, z, s.eps, mode=1))
    # group 3: per-head RMSNorm(1 + w) then partial RoPE at random positions
    q, k = synth.act("g.q", T, s.q_heads, s.head_dim), synth.act("g.k", T, s.kv_heads, s.head_dim)
    pos = synth.positions("g.pos", T, s.max_pos)
    qw, kw = synth.norm_w("g.qnorm_w", s.head_dim), synth.norm_w("g.knorm_w", s.head_dim)
    out.update(q=q, k=k, pos=pos, qnorm_w=qw, knorm_w=kw,
               q_rope=ref.rope_rows(q.copy(), pos, s.rot, s.theta), k_rope=ref.rope_rows(k.copy(), pos, s.rot, s.theta))
    qn = ref.rmsnorm_rows(q.copy(), np.float32(1.0) + qw, s.eps)
    kn = ref.rmsnorm_rows(k.copy(), np.float32(1.0) + kw, s.eps)
    out.update(q_norm_rope=ref.rope_rows(qn, pos, s.rot, s.theta), k_norm_rope=ref.rope_rows(kn, pos, s.rot, s.theta))
    # group 4: SwiGLU
    g, up = synth.act("g.gate", T, s.ff), synth.act("g.up", T, s.ff)
    out.update(gate=g, up=up, swiglu=ref.silu_mul(g.copy(), up))
    # group 5: Q8_0 embedding gather
    table = synth.q8_0_table("g.table", s.vocab, s.hidden)
    ids = synth.token_ids("g.ids", T, s.vocab)
    used = np.unique(ids)
    out.update(ids=ids, table_rows=used, table_bytes=table[used], embed=ref.embed_q8_0_rows(table, ids, s.hidden))
    return out


def make_wide_ops() -> dict:
    T = 12  # fewer tokens than the main fixture: these tensors are hc = 4 times wider
    ref = oracle.load("reference")
    assert ref.kind == "reference"
    s, hc, k, irows = synth.C1, 4, 3, 4
    out: dict[str, np.ndarray] = {}
    res, blk = synth.act("w.res", T, hc, s.hidden), synth.act("w.out", T, s.hidden)
    inject = synth.act("w.inject", T, hc) * 2
    gamma = (np.float32(1.0) + np.float32(0.1) * synth.act("w.gamma", hc, s.hidden)).astype(np.float32)
    out.update(hc_res=res, hc_out=blk, hc_inject=inject, hc_gamma=gamma)
    for name, rnd in (("f32", 0), ("bf16", 1), ("f16", 2)):
        r = res.copy()
        if rnd == 1:
            r = oracle.round_bf16(r)
        if rnd == 2:
            r = r.astype(np.float16).astype(np.float32)
        y = ref.hc_combine_norm(r, blk, inject, gamma, s.eps, rnd)
        out[f"hc_res_out_{name}"], out[f"hc_y_{name}"] = r, y
    iw = (synth.act("w.iw", irows, hc * s.hidden) * 0.05).astype(np.float32)
    out.update(hc_iw=iw, hc_inject_proj=ref.hc_inject(out["hc_y_f32"].reshape(T, -1), iw))
    gate = synth.act("w.gate", T, hc, s.hidden) * 2
    out.update(hc_gate=gate, hc_mixed=ref.hc_mix(out["hc_y_f32"], gate))
    yp = synth.act("w.yp", T * k, s.hidden).astype(np.float16).astype(np.float32)
    pos = synth.rng("w.pos").permutation(T * k).reshape(T, k).astype(np.uint32)
    mw = synth.rng("w.mw").random((T, k), dtype=np.float32)
    sx, sg = synth.act("w.sx", T, s.hidden), synth.act("w.sg", T)
    out.update(moe_yp=yp, moe_pos=pos, moe_w=mw, moe_sx=sx, moe_sg=sg, moe_routed=ref.moe_combine(yp, pos, mw),
               moe_out=ref.moe_combine(yp, pos, mw, sx, sg))
    C, l2 = (2 * s.k_heads + s.v_heads) * s.lin_dim, 2 * s.k_heads * s.lin_dim
    cx, cstate = synth.act("w.conv_x", T, C), synth.act("w.conv_state", 3, C)
    cw = (synth.act("w.conv_w", C, 4) * 0.5).astype(np.float32)
    st = cstate.copy()
    out.update(conv_x=cx, conv_state=cstate, conv_w=cw, conv_out=ref.conv_l2norm(cx, st, cw, l2, s.lin_dim, s.eps),
               conv_state_out=st)
    return out


if __name__ == "__main__":
    n = extract_quant_blocks()
    ops = make_ops()
    np.savez_compressed(HERE / "ops_c1.npz", **ops)
    wide = make_wide_ops()
    np.savez_compressed(HERE / "ops_wide_c1.npz", **wide)
    print(f"quant_blocks.tsv: {n} rows; ops_c1.npz: {len(ops)} arrays, "
          f"{(HERE / 'ops_c1.npz').stat().st_size} bytes; ops_wide_c1.npz: {len(wide)} arrays, "
          f"{(HERE / 'ops_wide_c1.npz').stat().st_size} bytes")
