"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no dataset is involved anywhere on this path).

Everything is drawn from one numpy PCG64 stream per (seed, tag): activations
~N(0,1), zero-centred norm weights ~N(0,0.1) (applied as 1 + w), gated-norm
weights ~N(1,0.1), token ids uniform over the vocabulary, positions uniform over
the context, Q8_0 tables with int8 codes uniform in [-127,127] and finite fp16
scales (exponent field 8..16, random mantissa and sign - the range the
reference's GPU tests draw, tests/gpu/quant_gpu_test.cpp:46-51).
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass

import numpy as np

SEED = 20261125


@dataclass(frozen=True)
class Shapes:
    name: str
    hidden: int
    q_heads: int
    kv_heads: int
    head_dim: int
    rot: int
    theta: float
    v_heads: int      # DeltaNet value heads (gated norm rows per token)
    k_heads: int      # DeltaNet key heads (q and k L2-norm rows per token, each)
    lin_dim: int      # DeltaNet head dim
    ff: int           # SwiGLU intermediate (shared expert)
    top_k: int        # routed experts per token (0: dense MLP only)
    experts: int
    vocab: int
    max_pos: int
    eps: float = 1e-6

    @property
    def q8_row_bytes(self) -> int:
        return self.hidden // 32 * 34


# Tiny Flash-Next-shaped chain the CPU reference runs.
C1 = Shapes("c1-tiny", hidden=256, q_heads=4, kv_heads=2, head_dim=64, rot=16, theta=1e7, v_heads=4, k_heads=2,
            lin_dim=64, ff=128, top_k=0, experts=0, vocab=4096, max_pos=4096)
# Full-size layer: decode, T=4096 prefill and the 48-layer chain all use these dims.
FULL = Shapes("full", hidden=2048, q_heads=16, kv_heads=2, head_dim=256, rot=64, theta=1e7, v_heads=32, k_heads=16,
              lin_dim=128, ff=512, top_k=10, experts=512, vocab=151936, max_pos=262144)

# 48 layers, 3 DeltaNet : 1 GQA (every fourth layer is attention).
LAYERS = 48
def layer_is_gqa(layer: int) -> bool:
    return layer % 4 == 3


def rng(tag: str, seed: int = SEED) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64([seed, zlib.crc32(tag.encode())]))


def act(tag: str, *shape, seed: int = SEED) -> np.ndarray:
    return rng(tag, seed).standard_normal(shape, dtype=np.float32)


def norm_w(tag: str, d: int, seed: int = SEED) -> np.ndarray:
    return (0.1 * rng(tag, seed).standard_normal(d, dtype=np.float32)).astype(np.float32)


def gated_w(tag: str, d: int, seed: int = SEED) -> np.ndarray:
    return (1.0 + 0.1 * rng(tag, seed).standard_normal(d, dtype=np.float32)).astype(np.float32)


def token_ids(tag: str, n: int, vocab: int, seed: int = SEED) -> np.ndarray:
    return rng(tag, seed).integers(0, vocab, size=n, dtype=np.uint32)


def positions(tag: str, n: int, max_pos: int, seed: int = SEED) -> np.ndarray:
    return rng(tag, seed).integers(0, max_pos, size=n, dtype=np.uint32)


def q8_0_table(tag: str, vocab: int, cols: int, seed: int = SEED) -> np.ndarray:
    """uint8 [vocab, cols/32*34]: per block a little-endian fp16 scale then 32 int8 codes."""
    g = rng(tag, seed)
    nb = cols // 32
    codes = g.integers(-127, 128, size=(vocab, nb, 32), dtype=np.int8)
    exp = g.integers(8, 17, size=(vocab, nb), dtype=np.uint16)
    mant = g.integers(0, 1024, size=(vocab, nb), dtype=np.uint16)
    sign = g.integers(0, 2, size=(vocab, nb), dtype=np.uint16)
    scale = ((sign << 15) | (exp << 10) | mant).astype("<u2")
    table = np.empty((vocab, nb, 34), dtype=np.uint8)
    table[:, :, 0:2] = scale.view(np.uint8).reshape(vocab, nb, 2)
    table[:, :, 2:] = codes.view(np.uint8)
    return table.reshape(vocab, nb * 34)


def routed_assignments(tag: str, tokens: int, top_k: int, experts: int, seed: int = SEED) -> np.ndarray:
    """[tokens, top_k] distinct expert ids per token, uniform; row order pair = t * top_k + slot."""
    g = rng(tag, seed)
    keys = g.random((tokens, experts), dtype=np.float32)
    return np.argpartition(keys, top_k, axis=1)[:, :top_k].astype(np.uint32)
