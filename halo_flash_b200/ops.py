"""Tensor-level front end of the C ABI: the five op groups on torch CUDA tensors.

torch is plumbing here (device memory and the current stream); every function
forwards to one `halo_b200_*` entry point of libhalo_b200.so and nothing else.
CPU tensors are rejected: the CUDA library is the only implementation.

Conventions follow the reference kernels (src/kernels/core.hip): rows are the
leading dimensions flattened, the last dimension is `d`; in-place is the
default where the reference kernel is in-place.
"""
from __future__ import annotations

import torch

from ._lib import BF16, F16, F32, lib

_DT = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _chk(t: torch.Tensor | None, name: str, dtypes=None):
    if t is None:
        return None
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{name}: expected a CUDA tensor (halo_flash_b200 has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name}: tensor must be contiguous")
    if dtypes is not None and t.dtype not in dtypes:
        raise TypeError(f"{name}: dtype {t.dtype} not in {dtypes}")
    return t


def _p(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


_ACT = (torch.float32, torch.float16, torch.bfloat16)


# ---- group 1 ---------------------------------------------------------------
def rmsnorm(x, w, eps, *, y=None, one_plus=False, w_stride=0, w_period=1):
    """y = x * rsqrt(mean(x^2) + eps) * g per row, g = w or 1 + w. y defaults to x (in place)."""
    _chk(x, "x", _ACT), _chk(w, "w", (torch.float32,))
    y = x if y is None else _chk(y, "y", _ACT)
    d = x.shape[-1]
    rows = x.numel() // d if d else 0
    lib().call("rmsnorm_ex", _stream(), _p(x), _code(x), _p(w), _p(y), _code(y), d, eps, w_stride, w_period,
               int(one_plus), rows)
    return y


def add_rmsnorm(res, delta, w, eps, *, one_plus=True, xn=None, q8_0=None, xq=None, xd=None):
    """res += delta (stored in res' dtype); then RMSNorm of the stored rows into any of
    xn (fp32/fp16/bf16), q8_0 (uint8 [rows, d/32*34]), xq/xd (int8 codes + fp32 scales)."""
    _chk(res, "res", _ACT), _chk(delta, "delta", (res.dtype,)), _chk(w, "w", (torch.float32,))
    _chk(xn, "xn", _ACT), _chk(q8_0, "q8_0", (torch.uint8,)), _chk(xq, "xq", (torch.int8,))
    _chk(xd, "xd", (torch.float32,))
    d = res.shape[-1]
    rows = res.numel() // d if d else 0
    lib().call("add_rmsnorm", _stream(), _p(res), _p(delta), _code(res), _p(w), int(one_plus), _p(xn),
               _code(xn) if xn is not None else F32, _p(q8_0), _p(xq), _p(xd), d, eps, rows)
    return xn


def encode_q8_0(x, out):
    """Q8_0 rows (34-byte blocks) of x [rows, cols] into out uint8 [rows, cols/32*34]."""
    _chk(x, "x", _ACT), _chk(out, "out", (torch.uint8,))
    cols = x.shape[-1]
    lib().call("encode_q8_0_rows", _stream(), _p(x), _code(x), _p(out), cols, x.numel() // cols if cols else 0)
    return out


def quantize_q8_rows(x, xq, xd):
    _chk(x, "x", (torch.float32,)), _chk(xq, "xq", (torch.int8,)), _chk(xd, "xd", (torch.float32,))
    cols = x.shape[-1]
    lib().call("quantize_q8_rows", _stream(), _p(x), _p(xq), _p(xd), cols, x.numel() // cols if cols else 0)
    return xq, xd


# ---- group 2 ---------------------------------------------------------------
def l2norm(x, eps, *, y=None):
    """y = x * rsqrt(sum(x^2) + eps) per row (eps inside the root, on the sum)."""
    _chk(x, "x", _ACT)
    y = x if y is None else _chk(y, "y", _ACT)
    d = x.shape[-1]
    lib().call("l2norm_ex", _stream(), _p(x), _code(x), _p(y), _code(y), d, eps, x.numel() // d if d else 0)
    return y


def gated_norm(o, w, z, eps, *, mode=0, y=None):
    """y = RMSNorm(o; plain weight w[d]) * SiLU(z) (mode 0) or * sigmoid(z) (mode 1), per head row."""
    _chk(o, "o", _ACT), _chk(z, "z", _ACT), _chk(w, "w", (torch.float32,))
    y = o if y is None else _chk(y, "y", _ACT)
    d = o.shape[-1]
    lib().call("gated_norm_ex", _stream(), _p(o), _code(o), _p(w), _p(z), _code(z), _p(y), _code(y), d, eps, mode,
               o.numel() // d if d else 0)
    return y


# ---- group 3 ---------------------------------------------------------------
def rope(q, k, rot, theta, *, pos0=0, params=None, pstride=0, slot=0, scale=1, pos_out=None):
    """In-place partial NEOX RoPE on q [T, Hq, hd] and optionally k [T, Hk, hd].
    Token t rotates at (params[t*pstride+slot] if params is given else pos0 + t) * scale."""
    _chk(q, "q", _ACT), _chk(k, "k", (q.dtype,)), _chk(params, "params", (torch.int32, torch.uint32))
    _chk(pos_out, "pos_out", (torch.int32, torch.uint32))
    tokens, hq, hd = q.shape
    hk = 0 if k is None else k.shape[1]
    lib().call("rope_ex", _stream(), _p(q), hq, _p(k), hk, _code(q), hd, rot, theta, tokens, _p(params), pstride, slot,
               pos0, scale, _p(pos_out))
    return q, k


def norm_rope(x, w, eps, rot, theta, heads, *, out=None, gate=None, cache=None, one_plus=True, in_row_stride=None,
              pos0=0, params=None, pstride=0, slot=0, scale=1, pos_out=None):
    """Per-head RMSNorm (gamma w or 1 + w) fused with RoPE on rows [T * heads, d]."""
    _chk(x, "x", _ACT), _chk(w, "w", (torch.float32,))
    out = x if out is None else _chk(out, "out", _ACT)
    _chk(gate, "gate", (x.dtype,)), _chk(cache, "cache", (out.dtype,))
    d = out.shape[-1]
    rows = out.numel() // d if d else 0
    stride = d if in_row_stride is None else in_row_stride
    lib().call("norm_rope_ex", _stream(), _p(x), _code(x), stride, _p(out), _code(out), _p(gate), _p(cache), _p(w),
               int(one_plus), eps, d, rot, heads, rows, theta, _p(params), pstride, slot, pos0, scale, _p(pos_out))
    return out


def norm_rope_qk(q, k, w_q, w_k, eps, rot, theta, *, q_out=None, q_gate=None, k_cache=None, one_plus=True,
                 q_row_stride=None, pos0=0, params=None, pstride=0, slot=0, scale=1, pos_out=None):
    """Per-head RMSNorm + RoPE of Q [T, Hq, d] and K [T, Hk, d] in one launch (in place unless q_out is given)."""
    _chk(q, "q", _ACT), _chk(k, "k", (q.dtype,)), _chk(w_q, "w_q", (torch.float32,)), _chk(w_k, "w_k", (torch.float32,))
    q_out = q if q_out is None else _chk(q_out, "q_out", _ACT)
    _chk(q_gate, "q_gate", (q.dtype,)), _chk(k_cache, "k_cache", (q_out.dtype,))
    tokens, hq, d = q_out.shape
    hk = k.shape[1]
    stride = d if q_row_stride is None else q_row_stride
    lib().call("norm_rope_qk_ex", _stream(), _p(q), stride, _p(q_out), _p(q_gate), _p(w_q), hq, _p(k), _p(k), _p(k_cache),
               _p(w_k), hk, _code(q), _code(q_out), int(one_plus), eps, d, rot, tokens, theta, _p(params), pstride, slot,
               pos0, scale, _p(pos_out))
    return q_out, k


def rope_table(table, rot, theta, *, pos0=0, params=None, pstride=0, slot=0, scale=1, pos_out=None):
    """Fill table [T, 2, rot/2] fp32 with cos / sin of every token's rotation angles."""
    _chk(table, "table", (torch.float32,)), _chk(params, "params", (torch.int32, torch.uint32))
    _chk(pos_out, "pos_out", (torch.int32, torch.uint32))
    tokens = table.numel() // rot if rot else 0
    lib().call("rope_table_ex", _stream(), _p(table), tokens, rot, theta, _p(params), pstride, slot, pos0, scale,
               _p(pos_out))
    return table


def norm_rope_qk_table(q, k, w_q, w_k, eps, rot, table, *, q_out=None, q_gate=None, k_cache=None, one_plus=True,
                       q_row_stride=None):
    """norm_rope_qk with the rotation table of rope_table() (k may be None)."""
    _chk(q, "q", _ACT), _chk(k, "k", (q.dtype,)), _chk(w_q, "w_q", (torch.float32,)), _chk(w_k, "w_k", (torch.float32,))
    _chk(table, "table", (torch.float32,))
    q_out = q if q_out is None else _chk(q_out, "q_out", _ACT)
    _chk(q_gate, "q_gate", (q.dtype,)), _chk(k_cache, "k_cache", (q_out.dtype,))
    tokens, hq, d = q_out.shape
    hk = 0 if k is None else k.shape[1]
    stride = d if q_row_stride is None else q_row_stride
    lib().call("norm_rope_qk_table_ex", _stream(), _p(q), stride, _p(q_out), _p(q_gate), _p(w_q), hq, _p(k), _p(k),
               _p(k_cache), _p(w_k), hk, _code(q), _code(q_out), int(one_plus), eps, d, rot, tokens, _p(table))
    return q_out, k


# ---- group 4 ---------------------------------------------------------------
def silu_mul(g, up, *, y=None):
    """y = SiLU(g) * up elementwise; y defaults to g (in place)."""
    _chk(g, "g", _ACT), _chk(up, "up", (g.dtype,))
    y = g if y is None else _chk(y, "y", _ACT)
    lib().call("silu_mul_ex", _stream(), _p(g), _p(up), _code(g), _p(y), _code(y), g.numel())
    return y


def silu_mul_multi(pairs, outs):
    """SiLU(g) * up for several (g, up) -> y tensors in one launch (at most 4; same dtypes)."""
    import ctypes as C
    n = len(pairs)
    assert n == len(outs) and 1 <= n <= 4
    for (g, up), y in zip(pairs, outs):
        _chk(g, "g", _ACT), _chk(up, "up", (pairs[0][0].dtype,)), _chk(y, "y", (outs[0].dtype,))
        assert g.dtype == pairs[0][0].dtype and g.numel() == up.numel() == y.numel()
    arr = lambda vals: (C.c_void_p * n)(*vals)
    gs, us, ys = arr([g.data_ptr() for g, _ in pairs]), arr([u.data_ptr() for _, u in pairs]), arr([y.data_ptr() for y in outs])
    ns = (C.c_uint64 * n)(*[g.numel() for g, _ in pairs])
    lib().call("silu_mul_multi_ex", _stream(), n, gs, us, ys, ns, _code(pairs[0][0]), _code(outs[0]))
    return outs


# ---- group 5 ---------------------------------------------------------------
def embed_q8_0(table, ids, cols, out, *, id_stride=1, id_slot=0, vocab=0):
    """out[t] = dequant(table[ids[t*id_stride + id_slot]]); table uint8 [vocab, cols/32*34]."""
    _chk(table, "table", (torch.uint8,)), _chk(ids, "ids", (torch.int32, torch.uint32)), _chk(out, "out", _ACT)
    tokens = out.numel() // cols if cols else 0
    lib().call("embed_q8_0_ex", _stream(), _p(table), table.shape[-1], vocab, _p(ids), id_stride, id_slot, tokens,
               _p(out), _code(out), cols)
    return out


# ---- hyper-connection residual (hc streams of h values per token) -----------------------------
def hc_combine_norm(res, out, inject, w, eps, *, one_plus=False, y=None, y16=None, y16_tokens=0, rscale=None, iw=None,
                    ipart=None, yq=None, yd=None):
    """res [T, hc, h] += out [T, h] * 2 sigmoid(inject [T, hc] / hc), stored in res' dtype; then the
    grouped RMSNorm of the stored streams (gamma w [hc, h]) into any of y, y16 (fp16; K-blocked when
    y16_tokens > 0), rscale [T, hc], yq / yd (K-blocked int8 + scales), ipart [T, hc, irows] = partial
    products with iw [irows, hc*h]. out = inject = None: grouped norm only."""
    _chk(res, "res", _ACT), _chk(out, "out", _ACT), _chk(inject, "inject", (torch.float32,))
    _chk(w, "w", (torch.float32,)), _chk(y, "y", _ACT), _chk(y16, "y16", (torch.float16,))
    _chk(rscale, "rscale", (torch.float32,)), _chk(iw, "iw", (torch.float32,)), _chk(ipart, "ipart", (torch.float32,))
    _chk(yq, "yq", (torch.int8,)), _chk(yd, "yd", (torch.float32,))
    tokens, hc, h = res.shape
    lib().call("hc_combine_norm_ex", _stream(), _p(res), _code(res), _p(out), _code(out) if out is not None else F32,
               _p(inject), _p(w), int(one_plus), _p(y), _code(y) if y is not None else F32, _p(y16), y16_tokens,
               _p(rscale), _p(iw), _p(ipart), iw.shape[0] if iw is not None else 0, _p(yq), _p(yd), hc, h, eps, tokens)
    return y


def hc_combine_norm_moe(res, yp, pos, mw, sx, sg, inject, w, eps, *, one_plus=False, y=None, y16=None, y16_tokens=0,
                        rscale=None, iw=None, ipart=None):
    """hc_combine_norm whose block output is built in the kernel: sum over the k slots of
    mw[t, s] * yp[pos[t, s]] (expert output rows), then + sigmoid(sg[t]) * sx[t] (shared expert)."""
    _chk(res, "res", _ACT), _chk(yp, "yp", (torch.float16, torch.bfloat16)), _chk(pos, "pos", (torch.int32, torch.uint32))
    _chk(mw, "mw", (torch.float32,)), _chk(sx, "sx", (torch.float32, yp.dtype)), _chk(sg, "sg", (torch.float32,))
    _chk(inject, "inject", (torch.float32,)), _chk(w, "w", (torch.float32,)), _chk(y, "y", _ACT)
    _chk(y16, "y16", (torch.float16,)), _chk(rscale, "rscale", (torch.float32,)), _chk(iw, "iw", (torch.float32,))
    _chk(ipart, "ipart", (torch.float32,))
    tokens, hc, h = res.shape
    lib().call("hc_combine_norm_moe_ex", _stream(), _p(res), _code(res), _p(yp), _code(yp), _p(pos), _p(mw), _p(sx),
               _code(sx), _p(sg), pos.shape[1], _p(inject), _p(w), int(one_plus), _p(y),
               _code(y) if y is not None else F32, _p(y16), y16_tokens, _p(rscale), _p(iw), _p(ipart),
               iw.shape[0] if iw is not None else 0, hc, h, eps, tokens)
    return y


def hc_combine_rows(res, out, inject):
    """res [T, hc, h] += out [T, h] * 2 sigmoid(inject [T, hc] / hc)."""
    _chk(res, "res", _ACT), _chk(out, "out", _ACT), _chk(inject, "inject", (torch.float32,))
    tokens, hc, h = res.shape
    lib().call("hc_combine_rows_ex", _stream(), _p(res), _code(res), _p(out), _code(out), _p(inject), hc, h, tokens)
    return res


def broadcast_rows(res, x):
    """res [T, hc, h] = x [T, h] in every stream."""
    _chk(res, "res", _ACT), _chk(x, "x", _ACT)
    tokens, hc, h = res.shape
    lib().call("broadcast_rows_ex", _stream(), _p(res), _code(res), _p(x), _code(x), hc, h, tokens)
    return res


def hc_mix_rows(xn, gate, mixed):
    """mixed [T, h] = mean over streams of xn [T, hc, h] * sigmoid(gate [T, hc, h])."""
    _chk(xn, "xn", _ACT), _chk(gate, "gate", (xn.dtype,)), _chk(mixed, "mixed", (xn.dtype,))
    tokens, hc, h = xn.shape
    lib().call("hc_mix_rows_ex", _stream(), _p(xn), _p(gate), _p(mixed), _code(xn), hc, h, tokens)
    return mixed


def axpy_sigmoid_rows(y, x, g):
    """y [T, n] += sigmoid(g [T]) * x [T, n]."""
    _chk(y, "y", (torch.float32,)), _chk(x, "x", (torch.float32,)), _chk(g, "g", (torch.float32,))
    tokens, n = y.shape
    lib().call("axpy_sigmoid_rows", _stream(), _p(y), _p(x), _p(g), n, tokens)
    return y


def inject_reduce(ipart, inject):
    """inject [T, irows] = sum over streams of ipart [T, hc, irows]."""
    _chk(ipart, "ipart", (torch.float32,)), _chk(inject, "inject", (torch.float32,))
    tokens, hc, irows = ipart.shape
    lib().call("inject_reduce", _stream(), _p(ipart), _p(inject), hc, irows, tokens)
    return inject


# ---- Gated DeltaNet causal conv + SiLU + per-head L2 norm -------------------------------------
def conv_l2norm(x, state, w, out, *, l2_channels, d, eps):
    """out [T, C] = SiLU(causal depthwise conv of x [T, C] with taps w [C, kern]); history before the chunk
    from state [kern - 1, C] (fp32, oldest first; None = zeros). The first l2_channels channels are
    L2-normalized per head of d channels. The state is not written: see conv_state_advance."""
    _chk(x, "x", _ACT), _chk(state, "state", (torch.float32,)), _chk(w, "w", (torch.float32,)), _chk(out, "out", _ACT)
    tokens, channels = x.shape
    lib().call("conv_l2norm_ex", _stream(), _p(x), _code(x), _p(state), _p(w), _p(out), _code(out), channels, w.shape[1],
               l2_channels, d, eps, tokens)
    return out


def conv_state_advance(x, state):
    """state [kern - 1, C] <- the last kern - 1 rows of (state rows, then x rows)."""
    _chk(x, "x", _ACT), _chk(state, "state", (torch.float32,))
    tokens, channels = x.shape
    lib().call("conv_state_advance", _stream(), _p(x), _code(x), _p(state), channels, state.shape[0] + 1, tokens)
    return state


# ---- MoE combine ----------------------------------------------------------------------------------
def moe_combine(yp, pos, mw, out, *, sx=None, sg=None):
    """out [T, n] = sum over the k slots of mw[t, s] * yp[pos[t, s]] (+ sigmoid(sg[t]) * sx[t]).
    pos None: slot s of token t is row t*k + s of yp."""
    _chk(yp, "yp", _ACT), _chk(pos, "pos", (torch.int32, torch.uint32)), _chk(mw, "mw", (torch.float32,))
    _chk(out, "out", _ACT), _chk(sx, "sx", (torch.float32, yp.dtype)), _chk(sg, "sg", (torch.float32,))
    tokens, k = mw.shape
    n = out.shape[-1]
    lib().call("moe_combine_ex", _stream(), _p(yp), _code(yp), _p(pos), _p(mw), _p(sx), _code(sx) if sx is not None else F32,
               _p(sg), _p(out), _code(out), k, n, tokens)
    return out
