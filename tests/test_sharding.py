"""Host-side logic of token-sharded execution, on CPU: the shard arithmetic, and a world-size-2
`gloo` run in which each rank computes its own token shard with the CPU oracle, nothing is
exchanged on the data path, and the concatenated shards equal the unsharded result bit for bit
(RoPE positions offset by the shard's first token)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from halo_flash_b200 import chain, synth


def test_shard_ranges_cover_the_batch_exactly():
    for total in (0, 1, 7, 4096, 65536, 65537):
        for world in (1, 2, 3, 4, 8):
            spans = [chain.shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
                assert e0 == b1 and e0 >= b0
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def test_chain_byte_model_matches_the_per_op_table():
    """Algorithmic bytes per token of the full-size chain: 36 DeltaNet layers x 107520 B,
    12 GQA layers x (2 x 16384 + 18432 + 33792) B, plus the embedding row (6276 B)."""
    b = chain.bytes_per_token(synth.FULL, 2)
    assert b == {"add_rmsnorm": 16384, "l2norm": 16384, "gated_norm": 24576, "norm_rope": 18432,
                 "swiglu_shared": 3072, "swiglu_routed": 30720, "embed": 6276}
    assert chain.chain_bytes_per_token(synth.FULL, 2) == 36 * 107520 + 12 * 84992 + 6276


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _layer_ops(orc, s, res, delta, q, pos, g_h, g_q):
    """One GQA layer's token-local ops on a token range (CPU oracle)."""
    orc.add(res, delta)
    xn = orc.rmsnorm_rows(res.copy(), g_h, s.eps)
    qn = orc.rmsnorm_rows(q.reshape(-1, s.head_dim).copy(), g_q, s.eps).reshape(q.shape)
    orc.rope_rows(qn, pos, s.rot, s.theta)
    return xn, qn


def _worker(rank, world, port, T, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    orc = oracle.load("port")
    s = synth.C1
    b, e = chain.shard_range(T, rank, world)
    # every rank regenerates the same seeded global inputs and keeps only its token rows
    res, delta = synth.act("sh.res", T, s.hidden)[b:e].copy(), synth.act("sh.delta", T, s.hidden)[b:e].copy()
    q = synth.act("sh.q", T, s.q_heads, s.head_dim)[b:e].copy()
    g_h, g_q = np.float32(1) + synth.norm_w("sh.wh", s.hidden), np.float32(1) + synth.norm_w("sh.wq", s.head_dim)
    pos = np.arange(b, e, dtype=np.uint32) + np.uint32(1000)  # pos0 + global token index
    xn, qn = _layer_ops(orc, s, res, delta, q, pos, g_h, g_q)
    np.savez(os.path.join(out_dir, f"shard{rank}.npz"), xn=xn, qn=qn, res=res)
    # the only communication of the sharded path: a barrier and the max of the ranks' times
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == world
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_rank_token_sharding_equals_unsharded(tmp_path):
    import oracle
    T, world = 37, 2
    mp.spawn(_worker, args=(world, _free_port(), T, str(tmp_path)), nprocs=world, join=True)
    orc = oracle.load("port")
    s = synth.C1
    res, delta = synth.act("sh.res", T, s.hidden), synth.act("sh.delta", T, s.hidden)
    q = synth.act("sh.q", T, s.q_heads, s.head_dim)
    g_h, g_q = np.float32(1) + synth.norm_w("sh.wh", s.hidden), np.float32(1) + synth.norm_w("sh.wq", s.head_dim)
    xn, qn = _layer_ops(orc, s, res, delta, q, np.arange(T, dtype=np.uint32) + np.uint32(1000), g_h, g_q)
    parts = [np.load(tmp_path / f"shard{r}.npz") for r in range(world)]
    assert np.concatenate([p["xn"] for p in parts]).tobytes() == xn.tobytes()
    assert np.concatenate([p["qn"] for p in parts]).tobytes() == qn.tobytes()
    assert np.concatenate([p["res"] for p in parts]).tobytes() == res.tobytes()
