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
        torch.cuda.synchronize()
        # free device memory as the driver reports it (cudaMemGetInfo): unlike torch's own counters it moves
        # with any allocation made inside the library. The first call on a device only resolves the array's
        # address, so from the second call on the figure must not move at all.
        free_before, _ = torch.cuda.mem_get_info()
        _call("norm_rope_qk_noalloc", q_new, k_new, wq, wk, s, tokens, pos0, used_new)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        if call > 0:
            assert free_after == free_before, "the allocation-free entry point changed the device's free memory"
        assert torch.equal(q_new, q_ref) and torch.equal(k_new, k_ref), f"call {call}: results differ"
        assert torch.equal(used_new, used_ref)
        assert not torch.equal(q_new, _bf16(q)), "the op must have changed its input"


def test_noalloc_calls_of_alternating_sizes_on_one_stream_without_a_sync():
    """Calls on one stream are ordered even though they share the array: eight calls of alternating sizes and
    positions are enqueued back to back and only then compared with the allocating entry point."""
    s = synth.FULL
    wq = torch.from_numpy(synth.norm_w("na.wq", s.head_dim)).to(DEV)
    wk = torch.from_numpy(synth.norm_w("na.wk", s.head_dim)).to(DEV)
    cases = [(64 if i % 2 == 0 else 160, 1000 * i + 3) for i in range(8)]
    new, ref = [], []
    for i, (tokens, pos0) in enumerate(cases):
        q, k = synth.act(f"na.alt.q{i}", tokens, s.q_heads, s.head_dim), synth.act(f"na.alt.k{i}", tokens, s.kv_heads, s.head_dim)
        new.append((_bf16(q), _bf16(k), torch.zeros(tokens, dtype=torch.int32, device=DEV)))
        ref.append((_bf16(q), _bf16(k), torch.zeros(tokens, dtype=torch.int32, device=DEV)))
    torch.cuda.synchronize()
    for (tokens, pos0), (q, k, used) in zip(cases, new):
        _call("norm_rope_qk_noalloc", q, k, wq, wk, s, tokens, pos0, used)
    for (tokens, pos0), (q, k, used) in zip(cases, ref):
        _call("norm_rope_qk_ex", q, k, wq, wk, s, tokens, pos0, used)
    torch.cuda.synchronize()
    for i, (a, b) in enumerate(zip(new, ref)):
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]), f"call {i}"


def test_noalloc_failed_call_enqueues_nothing_and_odd_shapes_take_the_table_free_form():
    s = synth.FULL
    st = torch.cuda.current_stream().cuda_stream
    tokens = 8
    q = _bf16(synth.act("na.bad.q", tokens, s.q_heads, s.head_dim))
    k = _bf16(synth.act("na.bad.k", tokens, s.kv_heads, s.head_dim))
    w = torch.zeros(s.head_dim, device=DEV)
    used = torch.full((tokens,), -1, dtype=torch.int32, device=DEV)
    q0 = q.clone()
    # an invalid call (rotary_dim larger than d): refused before the table kernel could write pos_out
    with pytest.raises(HaloError, match="rotary_dim"):
        lib().call("norm_rope_qk_noalloc", st, q.data_ptr(), s.head_dim, q.data_ptr(), None, w.data_ptr(), s.q_heads,
                   k.data_ptr(), k.data_ptr(), None, w.data_ptr(), s.kv_heads, BF16, BF16, 1, s.eps, s.head_dim,
                   s.head_dim + 2, tokens, s.theta, None, 0, 0, 5, 1, used.data_ptr())
    torch.cuda.synchronize()
    assert bool((used == -1).all()) and torch.equal(q, q0), "a refused call must not have launched anything"
    # rows that are not 16-byte aligned cannot use a table: the call still works (Q only, fp32, d = 20, rot = 6)
    heads, d, rot = 2, 20, 6
    x = synth.act("na.odd.x", tokens, heads, d)
    wq = torch.from_numpy(synth.norm_w("na.odd.w", d)).to(DEV)
    a, b = torch.from_numpy(x).to(DEV), torch.from_numpy(x).to(DEV)
    for name, t in (("norm_rope_qk_noalloc", a), ("norm_rope_qk_ex", b)):
        lib().call(name, st, t.data_ptr(), d, t.data_ptr(), None, wq.data_ptr(), heads, None, None, None, None, 0, 0, 0, 1,
                   s.eps, d, rot, tokens, s.theta, None, 0, 0, 11, 1, None)
    torch.cuda.synchronize()
    assert torch.equal(a, b) and not torch.equal(a, torch.from_numpy(x).to(DEV))


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
