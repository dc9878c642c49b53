"""Generates the committed golden fixtures. Run in a container that has the
reference checkout (default /root/reference):

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


if __name__ == "__main__":
    n = extract_quant_blocks()
    ops = make_ops()
    np.savez_compressed(HERE / "ops_c1.npz", **ops)
    print(f"quant_blocks.tsv: {n} rows; ops_c1.npz: {len(ops)} arrays, "
          f"{(HERE / 'ops_c1.npz').stat().st_size} bytes")
