"""The allocation-free entry point (GPU only; collected last on purpose).

halo_b200_norm_rope_qk_noalloc serves callers that may not allocate device memory - an engine
whose memory was fully committed and accounted for at load time, a serving loop that cannot take
cudaMalloc's device-wide synchronisation - by keeping the rotation table in a fixed array inside
the library. It must produce exactly what halo_b200_norm_rope_qk_ex produces, call after call
(the array keeps the previous call's table), and refuse sizes beyond its fixed array.
"""
import numpy as np
import pytest
import torch

from halo_flash_b200 import HaloError, lib, synth
from halo_flash_b200._lib import BF16

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _bf16(a):
    import oracle
    return torch.from_numpy(oracle.bf16_bits(a).view(np.int16)).to(DEV).view(torch.bfloat16).reshape(a.shape)


def _call(name, q, k, wq, wk, s, tokens, pos0, pos_out):
    st = torch.cuda.current_stream().cuda_stream
    lib().call(name, st, q.data_ptr(), s.head_dim, q.data_ptr(), None, wq.data_ptr(), s.q_heads, k.data_ptr(),
               k.data_ptr(), None, wk.data_ptr(), s.kv_heads, BF16, BF16, 1, s.eps, s.head_dim, s.rot, tokens, s.theta,
               None, 0, 0, pos0, 1, pos_out.data_ptr())


def test_noalloc_entry_point_matches_the_allocating_one_twice_in_a_row():
    s = synth.FULL
    wq = torch.from_numpy(synth.norm_w("na.wq", s.head_dim)).to(DEV)
    wk = torch.from_numpy(synth.norm_w("na.wk", s.head_dim)).to(DEV)
    # two calls in a row with different sizes and positions: the second must not see the first's table
    for call, (tokens, pos0) in enumerate(((96, 262144 - 96), (33, 7))):
        q = synth.act(f"na.q{call}", tokens, s.q_heads, s.head_dim)
        k = synth.act(f"na.k{call}", tokens, s.kv_heads, s.head_dim)
        q_ref, k_ref, q_new, k_new = _bf16(q), _bf16(k), _bf16(q), _bf16(k)
        used_ref = torch.zeros(tokens, dtype=torch.int32, device=DEV)
        used_new = torch.zeros(tokens, dtype=torch.int32, device=DEV)
        _call("norm_rope_qk_ex", q_ref, k_ref, wq, wk, s, tokens, pos0, used_ref)
        before = torch.cuda.memory_allocated()
        _call("norm_rope_qk_noalloc", q_new, k_new, wq, wk, s, tokens, pos0, used_new)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(q_new, q_ref) and torch.equal(k_new, k_ref), f"call {call}: results differ"
        assert torch.equal(used_new, used_ref)
        assert not torch.equal(q_new, _bf16(q)), "the op must have changed its input"


def test_noalloc_entry_point_refuses_tables_beyond_its_fixed_array():
    s = synth.FULL
    tokens = (1 << 20) // s.rot + 1  # one token too many for the 1 Mi-float array
    dummy = torch.zeros(8, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(s.head_dim, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    with pytest.raises(HaloError, match="exceeds the built-in scratch"):
        lib().call("norm_rope_qk_noalloc", st, dummy.data_ptr(), s.head_dim, dummy.data_ptr(), None, w.data_ptr(),
                   s.q_heads, dummy.data_ptr(), dummy.data_ptr(), None, w.data_ptr(), s.kv_heads, BF16, BF16, 1, s.eps,
                   s.head_dim, s.rot, tokens, s.theta, None, 0, 0, 0, 1, None)
    # nothing was launched: the device is idle and healthy
    torch.cuda.synchronize()
