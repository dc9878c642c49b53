"""The per-layer elementwise op chain of a 48-layer model (36 Gated-DeltaNet + 12 GQA
layers, 3:1) over one token shard, driven through the C ABI.

One step = embedding gather for the shard's tokens, then for every layer the ops that
sit between the projections of the reference's Qwen3.5 graph (src/model/qwen35.cpp:301-337;
engine order src/engine/qwen35_gpu.cpp:439-589):

    add + RMSNorm(1+w)                      res += previous block's output; xn = norm(res)
    DeltaNet layer : q/k L2 norm, gated RMSNorm of the recurrence output     (qwen35.cpp:196-197, 232-234)
    GQA layer      : per-head RMSNorm(1+w) + partial RoPE on Q and K, one fused launch (qwen35.cpp:251-255)
    add + RMSNorm(1+w)                      res += mixer output; xn = norm(res)
    SwiGLU on the shared-expert and on the routed-expert gate/up rows, one launch (qwen35.cpp:327)

The projections, the recurrence and attention between these ops are not part of the path;
their outputs are synthetic device tensors (the "block outputs" below). Only the residual
stream carries data from op to op. Block outputs live in `sets` rotating buffer sets so
that a layer never finds its inputs in L2 from the previous layer.

Token sharding: shard g of G owns tokens [g*T, (g+1)*T) and rotates at positions pos0 + t;
all ops are row-local, so shards exchange nothing.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops, synth
from .synth import Shapes


def shard_range(total_tokens: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous token range [begin, end) of shard `rank`; the first total % world shards get one extra token."""
    base, extra = divmod(total_tokens, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def bytes_per_token(s: Shapes, act_bytes: int = 2) -> dict[str, int]:
    """Algorithmic HBM bytes per token of each op (reads + writes of activations; gammas and the
    inverse-frequency table are cache-resident and excluded)."""
    H, a = s.hidden, act_bytes
    k = max(s.top_k, 0)
    return {
        "add_rmsnorm": 4 * a * H,                                   # read res, delta; write res, xn
        "l2norm": 2 * a * 2 * s.k_heads * s.lin_dim,               # q and k heads, in place
        "gated_norm": 3 * a * s.v_heads * s.lin_dim,               # read o, z; write y
        "norm_rope": 2 * a * (s.q_heads + s.kv_heads) * s.head_dim,  # q and k rows, in place
        "swiglu_shared": 3 * a * s.ff,
        "swiglu_routed": 3 * a * s.ff * k,
        "embed": s.q8_row_bytes + a * H + 4,
    }


def chain_bytes_per_token(s: Shapes, act_bytes: int = 2) -> int:
    b = bytes_per_token(s, act_bytes)
    n_gqa = sum(synth.layer_is_gqa(l) for l in range(synth.LAYERS))
    n_lin = synth.LAYERS - n_gqa
    mlp = b["swiglu_shared"] + b["swiglu_routed"]
    lin = 2 * b["add_rmsnorm"] + b["l2norm"] + b["gated_norm"] + mlp
    gqa = 2 * b["add_rmsnorm"] + b["norm_rope"] + mlp
    return n_lin * lin + n_gqa * gqa + b["embed"]


@dataclass
class BlockOutputs:
    """Synthetic outputs of the out-of-scope blocks of one layer (one rotating buffer set)."""
    delta_a: torch.Tensor   # [T, H]      previous MLP output
    delta_b: torch.Tensor   # [T, H]      mixer output
    qk: torch.Tensor        # [T, 2*k_heads, lin_dim]   conv output (q, k) before the L2 norm
    o: torch.Tensor         # [T*v_heads, lin_dim]      recurrence output
    z: torch.Tensor         # [T*v_heads, lin_dim]      output gate
    y: torch.Tensor         # [T*v_heads, lin_dim]      gated-norm result
    q: torch.Tensor         # [T, q_heads, head_dim]
    k: torch.Tensor         # [T, kv_heads, head_dim]
    gate_s: torch.Tensor    # [T, ff]
    up_s: torch.Tensor
    gate_r: torch.Tensor    # [T*top_k, ff]
    up_r: torch.Tensor

    def inputs(self):
        return [self.delta_a, self.delta_b, self.qk, self.o, self.z, self.q, self.k, self.gate_s, self.up_s,
                self.gate_r, self.up_r]


class LayerChain:
    def __init__(self, shapes: Shapes, tokens: int, *, pos0: int = 0, device="cuda:0", dtype=torch.bfloat16,
                 sets: int = 2, vocab: int | None = None, seed: int = synth.SEED, step_params: bool = False,
                 q8_epilogue: bool = False, rotate_outputs: bool = False):
        if not torch.cuda.is_available():
            raise RuntimeError("LayerChain needs a CUDA device: halo_flash_b200 has no CPU path")
        self.s, self.T, self.pos0, self.dtype = shapes, tokens, pos0, dtype
        self.device = torch.device(device)
        self.vocab = vocab or shapes.vocab
        s, T, dev = shapes, tokens, self.device
        g = torch.Generator(device=dev).manual_seed(seed + pos0)
        self._gen = g

        def act(*shape):
            return torch.randn(*shape, device=dev, generator=g, dtype=torch.float32).to(dtype)

        k = max(s.top_k, 1)
        self.sets = [BlockOutputs(
            delta_a=act(T, s.hidden), delta_b=act(T, s.hidden),
            qk=act(T, 2 * s.k_heads, s.lin_dim),
            o=act(T * s.v_heads, s.lin_dim), z=act(T * s.v_heads, s.lin_dim),
            y=torch.empty(T * s.v_heads, s.lin_dim, device=dev, dtype=dtype),
            q=act(T, s.q_heads, s.head_dim), k=act(T, s.kv_heads, s.head_dim),
            gate_s=act(T, s.ff), up_s=act(T, s.ff), gate_r=act(T * k, s.ff), up_r=act(T * k, s.ff),
        ) for _ in range(sets)]
        self.res = torch.empty(T, s.hidden, device=dev, dtype=dtype)
        self.xn = torch.empty(T, s.hidden, device=dev, dtype=dtype)
        # decode form of the add + norm: the normalized row leaves as Q8_0 blocks, the next GEMV's input
        self.xn_q8 = torch.empty(T, s.q8_row_bytes, device=dev, dtype=torch.uint8) if q8_epilogue else None
        self.h_s = torch.empty(T, s.ff, device=dev, dtype=dtype)
        self.h_r = torch.empty(T * k, s.ff, device=dev, dtype=dtype)
        # Measurement variant: the normalized rows and the SwiGLU outputs rotate through four buffers each, so
        # that no output line is overwritten while it still sits dirty in L2 (the default writes each into one
        # buffer, as an engine does with its scratch arena).
        self.out_ring = None
        if rotate_outputs:
            self.out_ring = [(torch.empty_like(self.xn), torch.empty_like(self.h_s), torch.empty_like(self.h_r))
                             for _ in range(4)]
        self.rope_tab = torch.empty(T, 2, s.rot // 2, device=dev, dtype=torch.float32)
        # weights: zero-centred norm gammas (applied as 1 + w), plain gated-norm gamma
        wg = torch.Generator(device="cpu").manual_seed(seed)
        def nw(d, mean=0.0):
            return (mean + 0.1 * torch.randn(d, generator=wg)).to(dev)
        self.w_attn = [nw(s.hidden) for _ in range(synth.LAYERS)]
        self.w_post = [nw(s.hidden) for _ in range(synth.LAYERS)]
        self.w_q, self.w_k = nw(s.head_dim), nw(s.head_dim)
        self.w_gated = nw(s.lin_dim, 1.0)
        # Q8_0 embedding table: int8 codes uniform, finite fp16 scales (exponent field 8..16)
        nb = s.hidden // 32
        codes = torch.randint(-127, 128, (self.vocab, nb, 32), device=dev, generator=g, dtype=torch.int8)
        half = (torch.randint(8, 17, (self.vocab, nb), device=dev, generator=g, dtype=torch.int32) << 10) | \
            torch.randint(0, 1024, (self.vocab, nb), device=dev, generator=g, dtype=torch.int32) | \
            (torch.randint(0, 2, (self.vocab, nb), device=dev, generator=g, dtype=torch.int32) << 15)
        table = torch.empty(self.vocab, nb, 34, device=dev, dtype=torch.uint8)
        table[:, :, 0] = (half & 0xFF).to(torch.uint8)
        table[:, :, 1] = ((half >> 8) & 0xFF).to(torch.uint8)
        table[:, :, 2:] = codes.view(torch.uint8)
        self.table = table.view(self.vocab, nb * 34)
        del codes, half, table
        self.ids = torch.randint(0, self.vocab, (T,), device=dev, generator=g, dtype=torch.int32)
        # Decode form: token and position of every batch entry live in device memory, rows 16 uint32 apart
        # (slot 0 = token, slot 1 = position: src/kernels/step_params.h), so a captured step replays at any
        # position after the host rewrites this buffer.
        self.params = None
        if step_params:
            self.params = torch.zeros(T, 16, device=dev, dtype=torch.int32)
            self.params[:, 0] = self.ids
            self.params[:, 1] = torch.arange(pos0, pos0 + T, device=dev, dtype=torch.int32)
        self.launches_per_step = 2 + 4 * synth.LAYERS + sum(not synth.layer_is_gqa(l) for l in range(synth.LAYERS))
        self._graph: torch.cuda.CUDAGraph | None = None

    # ---- one step, eager ------------------------------------------------------------------
    def layer(self, l: int, bo: BlockOutputs) -> None:
        s = self.s
        xn_a = xn_b = None if self.xn_q8 is not None else self.xn
        h_s, h_r = self.h_s, self.h_r
        if self.out_ring is not None and self.xn_q8 is None:
            xn_a, h_s, h_r = self.out_ring[(2 * l) % 4]
            xn_b = self.out_ring[(2 * l + 1) % 4][0]
        ops.add_rmsnorm(self.res, bo.delta_a, self.w_attn[l], s.eps, one_plus=True, xn=xn_a, q8_0=self.xn_q8)
        if synth.layer_is_gqa(l):
            ops.norm_rope_qk_table(bo.q, bo.k, self.w_q, self.w_k, s.eps, s.rot, self.rope_tab, one_plus=True)
        else:
            ops.l2norm(bo.qk, s.eps)
            ops.gated_norm(bo.o, self.w_gated, bo.z, s.eps, mode=0, y=bo.y)
        ops.add_rmsnorm(self.res, bo.delta_b, self.w_post[l], s.eps, one_plus=True, xn=xn_b, q8_0=self.xn_q8)
        ops.silu_mul_multi([(bo.gate_s, bo.up_s), (bo.gate_r, bo.up_r)], [h_s, h_r])

    def step(self) -> None:
        """Enqueue one full step on the current stream: the embedding gather and the rotation table,
        then per DeltaNet layer 5 launches (add+norm, L2, gated norm, add+norm, SwiGLU shared+routed)
        and per GQA layer 4 (add+norm, Q/K norm+RoPE, add+norm, SwiGLU): 2 + 36*5 + 12*4 = 230."""
        # every GQA layer rotates at the same positions: one cos / sin table per step
        if self.params is not None:
            ops.embed_q8_0(self.table, self.params, self.s.hidden, self.res, id_stride=16, id_slot=0, vocab=self.vocab)
            ops.rope_table(self.rope_tab, self.s.rot, self.s.theta, params=self.params, pstride=16, slot=1)
        else:
            ops.embed_q8_0(self.table, self.ids, self.s.hidden, self.res, vocab=self.vocab)
            ops.rope_table(self.rope_tab, self.s.rot, self.s.theta, pos0=self.pos0)
        for l in range(synth.LAYERS):
            self.layer(l, self.sets[l % len(self.sets)])

    # ---- one step, as a captured graph --------------------------------------------------------
    def capture(self) -> None:
        self.step()  # warm the allocator-free path once (ops allocate nothing, torch might)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        self._graph = g

    def replay(self) -> None:
        self._graph.replay()

    @property
    def step_bytes(self) -> int:
        return chain_bytes_per_token(self.s, self.res.element_size()) * self.T
