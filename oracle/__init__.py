"""ctypes bindings for the CPU checkers. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference
legs may import this package; the product (halo_flash_b200) never does.

Two libraries export the same ``orc_*`` C functions:

* ``port``      oracle/libhalo_oracle.so  - this repo's restatement (halo_oracle.cpp)
* ``reference`` oracle/_ref/libhalo_ref.so - halo-flash's own sources compiled
  unmodified (ref_shim.cpp only loops and forwards)

``load("port")`` / ``load("reference")`` return an :class:`Oracle`; ``best()``
prefers the compiled reference and falls back to the port. All array
arguments are C-contiguous numpy arrays; in-place functions modify and
return their first argument.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_LIB = HERE / "libhalo_oracle.so"
REF_LIB = HERE / "_ref" / "libhalo_ref.so"
# The halo-flash checkout: $HALO_REFERENCE_ROOT, else a directory named `reference` beside this repository.
REFERENCE_ROOT = Path(os.environ.get("HALO_REFERENCE_ROOT") or HERE.parent.parent / "reference")

_sz, _u32, _f32, _int, _p = C.c_size_t, C.c_uint32, C.c_float, C.c_int, C.c_void_p

_SIGS = {
    "orc_kind": (C.c_char_p, []),
    "orc_fp16_to_float": (_f32, [C.c_uint16]),
    "orc_bf16_to_float": (_f32, [C.c_uint16]),
    "orc_float_to_bf16": (C.c_uint16, [_f32]),
    "orc_float_to_fp16": (C.c_uint16, [_f32]),
    "orc_sigmoid": (_f32, [_f32]),
    "orc_silu": (_f32, [_f32]),
    "orc_add": (None, [_p, _p, _sz, _int]),
    "orc_rmsnorm_rows": (None, [_p, _p, _sz, _sz, _f32, _sz, _sz, _int]),
    "orc_l2norm_rows": (None, [_p, _sz, _sz, _f32, _int]),
    "orc_gated_norm_rows": (None, [_p, _p, _p, _sz, _sz, _f32, _u32, _int]),
    "orc_rope_rows": (None, [_p, _sz, _u32, _u32, _u32, _p, _f32, _int]),
    "orc_rope_inv_freq": (None, [_p, _u32, _f32]),
    "orc_silu_mul": (None, [_p, _p, _sz, _int]),
    "orc_embed_q8_0_rows": (None, [_p, _p, _sz, _sz, _sz, _p, _int]),
    "orc_dequant_f16": (None, [_p, _p, _sz]),
    "orc_dequant_bf16": (None, [_p, _p, _sz]),
    "orc_encode_q8_0_rows": (None, [_p, _sz, _sz, _p, _int]),
    "orc_quantize_i8_rows": (None, [_p, _sz, _sz, _p, _p, _int]),
    "orc_round_bf16": (None, [_p, _sz]),
    "orc_round_fp16": (None, [_p, _sz]),
    "orc_hc_combine_norm": (None, [_p, _p, _p, _p, _p, _sz, _sz, _sz, _f32, _int, _int]),
    "orc_hc_inject": (None, [_p, _p, _p, _sz, _sz, _sz, _int]),
    "orc_hc_mix": (None, [_p, _p, _p, _sz, _sz, _sz, _int]),
    "orc_conv_l2norm": (None, [_p, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _f32]),
    "orc_moe_combine": (None, [_p, _p, _p, _p, _p, _p, _sz, _sz, _sz, _int]),
}


def build(ref: bool | None = None) -> None:
    """Compile the port, and the reference library when its checkout is present."""
    targets = ["port"]
    if ref is None:
        ref = (REFERENCE_ROOT / "src" / "model" / "cpu_ops.cpp").exists()
    if ref:
        targets.append("ref")
    subprocess.run(["make", "-s", "-C", str(HERE), f"REF={REFERENCE_ROOT}", *targets], check=True)


def _f32arr(a, writable=False):
    a = np.ascontiguousarray(a, dtype=np.float32) if not writable else a
    if writable:
        assert a.dtype == np.float32 and a.flags.c_contiguous and a.flags.writeable, "need writable C-contiguous float32"
    return a


def _ptr(a):
    return a.ctypes.data_as(_p)


class Oracle:
    """One loaded checker library; `fallback` supplies functions the library lacks."""

    def __init__(self, path: Path, fallback: "Oracle | None" = None):
        self.path = Path(path)
        self._lib = C.CDLL(str(path))
        self._fallback = fallback
        self._fn = {}
        for name, (res, args) in _SIGS.items():
            try:
                f = getattr(self._lib, name)
            except AttributeError:
                continue
            f.restype, f.argtypes = res, args
            self._fn[name] = f
        self.kind = self._fn["orc_kind"]().decode()

    def has(self, name: str) -> bool:
        return name in self._fn

    def _call(self, name, *args):
        if name in self._fn:
            return self._fn[name](*args)
        if self._fallback is not None:
            return self._fallback._call(name, *args)
        raise AttributeError(f"{self.path.name} does not export {name}")

    # --- scalar helpers -------------------------------------------------
    def fp16_to_float(self, h: int) -> float:
        return self._call("orc_fp16_to_float", h)

    def bf16_to_float(self, h: int) -> float:
        return self._call("orc_bf16_to_float", h)

    # --- row operators (in place on float32 arrays) ------------------------
    def add(self, y, x, threads=1):
        y = _f32arr(y, True)
        x = _f32arr(x)
        assert x.size == y.size
        self._call("orc_add", _ptr(y), _ptr(x), y.size, threads)
        return y

    def rmsnorm_rows(self, x, g, eps, w_stride=0, w_period=1, threads=1):
        """x [rows, d] in place; g is the gamma actually multiplied (pass 1+w for a zero-centred weight)."""
        x = _f32arr(x, True)
        rows, d = x.reshape(-1, x.shape[-1]).shape
        gp = None
        if g is not None:
            g = _f32arr(g)
            gp = _ptr(g)
        self._call("orc_rmsnorm_rows", _ptr(x), gp, rows, d, eps, w_stride, w_period, threads)
        return x

    def l2norm_rows(self, x, eps, threads=1):
        x = _f32arr(x, True)
        rows, d = x.reshape(-1, x.shape[-1]).shape
        self._call("orc_l2norm_rows", _ptr(x), rows, d, eps, threads)
        return x

    def gated_norm_rows(self, o, w, z, eps, mode=0, threads=1):
        o = _f32arr(o, True)
        w = _f32arr(w)
        z = _f32arr(z)
        rows, d = o.reshape(-1, o.shape[-1]).shape
        assert z.size == o.size and w.size >= d
        self._call("orc_gated_norm_rows", _ptr(o), _ptr(w), _ptr(z), rows, d, eps, mode, threads)
        return o

    def rope_rows(self, x, pos, rot, theta, threads=1):
        """x [T, heads, hd] in place; pos [T] uint32."""
        x = _f32arr(x, True)
        tokens, heads, hd = x.shape
        pos = np.ascontiguousarray(pos, dtype=np.uint32)
        assert pos.size == tokens
        self._call("orc_rope_rows", _ptr(x), tokens, heads, hd, rot, _ptr(pos), theta, threads)
        return x

    def rope_inv_freq(self, rot, theta):
        out = np.empty(rot // 2, dtype=np.float32)
        self._call("orc_rope_inv_freq", _ptr(out), rot, theta)
        return out

    def silu_mul(self, g, up, threads=1):
        g = _f32arr(g, True)
        up = _f32arr(up)
        assert up.size == g.size
        self._call("orc_silu_mul", _ptr(g), _ptr(up), g.size, threads)
        return g

    def embed_q8_0_rows(self, table, ids, cols, threads=1):
        """table: uint8 [vocab, cols/32*34]; ids uint32 [T] -> float32 [T, cols]."""
        table = np.ascontiguousarray(table, dtype=np.uint8)
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        row_bytes = cols // 32 * 34
        out = np.empty((ids.size, cols), dtype=np.float32)
        self._call("orc_embed_q8_0_rows", _ptr(table), _ptr(ids), ids.size, cols, row_bytes, _ptr(out), threads)
        return out

    def dequant_f16(self, raw):
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.empty(raw.size // 2, dtype=np.float32)
        self._call("orc_dequant_f16", _ptr(raw), _ptr(out), out.size)
        return out

    def dequant_bf16(self, raw):
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.empty(raw.size // 2, dtype=np.float32)
        self._call("orc_dequant_bf16", _ptr(raw), _ptr(out), out.size)
        return out

    def encode_q8_0_rows(self, x, threads=1):
        """float32 [rows, cols] -> uint8 [rows, cols/32*34]."""
        x = _f32arr(x)
        rows, cols = x.reshape(-1, x.shape[-1]).shape
        out = np.empty((rows, cols // 32 * 34), dtype=np.uint8)
        self._call("orc_encode_q8_0_rows", _ptr(x), rows, cols, _ptr(out), threads)
        return out

    def quantize_i8_rows(self, x, threads=1):
        """float32 [rows, cols] -> (int8 [rows, cols], float32 [rows, cols/32]); fp32 scales, rint."""
        x = _f32arr(x)
        rows, cols = x.reshape(-1, x.shape[-1]).shape
        xq = np.empty((rows, cols), dtype=np.int8)
        xd = np.empty((rows, cols // 32), dtype=np.float32)
        self._call("orc_quantize_i8_rows", _ptr(x), rows, cols, _ptr(xq), _ptr(xd), threads)
        return xq, xd

    # --- hyper-connection residual --------------------------------------------
    def hc_combine_norm(self, res, out, inject, w, eps, round=0, threads=1):
        """res [T, hc, h] updated in place (out None: left as is), returns y = grouped norm of the stored res.
        round: 0 fp32 residual, 1 bf16, 2 fp16 storage."""
        res = _f32arr(res, True)
        tokens, hc, h = res.shape
        w = _f32arr(w)
        y = np.empty_like(res)
        op = ip = None
        if out is not None:
            out, inject = _f32arr(out), _f32arr(inject)
            assert out.size == tokens * h and inject.size == tokens * hc
            op, ip = _ptr(out), _ptr(inject)
        self._call("orc_hc_combine_norm", _ptr(res), op, ip, _ptr(w), _ptr(y), tokens, hc, h, eps, round, threads)
        return y

    def hc_inject(self, xn, iw, threads=1):
        """xn [T, hc*h], iw [irows, hc*h] -> inject [T, irows]."""
        xn, iw = _f32arr(xn), _f32arr(iw)
        tokens, cols = xn.reshape(xn.shape[0], -1).shape
        irows = iw.shape[0]
        out = np.empty((tokens, irows), dtype=np.float32)
        self._call("orc_hc_inject", _ptr(xn), _ptr(iw), _ptr(out), tokens, cols, irows, threads)
        return out

    def hc_mix(self, xn, gate, threads=1):
        xn, gate = _f32arr(xn), _f32arr(gate)
        tokens, hc, h = xn.shape
        out = np.empty((tokens, h), dtype=np.float32)
        self._call("orc_hc_mix", _ptr(xn), _ptr(gate), _ptr(out), tokens, hc, h, threads)
        return out

    def moe_combine(self, yp, pos, mw, sx=None, sg=None, threads=1):
        """sx / sg None: the routed experts' sum only."""
        yp, mw = _f32arr(yp), _f32arr(mw)
        pos = np.ascontiguousarray(pos, dtype=np.uint32)
        tokens, k = pos.shape
        h = yp.shape[-1]
        out = np.empty((tokens, h), dtype=np.float32)
        sp = gp = None
        if sx is not None:
            sx, sg = _f32arr(sx), _f32arr(sg)
            sp, gp = _ptr(sx), _ptr(sg)
        self._call("orc_moe_combine", _ptr(yp), _ptr(pos), _ptr(mw), sp, gp, _ptr(out), tokens, k, h, threads)
        return out

    def conv_l2norm(self, x, state, w, l2_channels, d, eps):
        """x [T, C], state [kern-1, C] (updated in place), w [C, kern] -> out [T, C]."""
        x, w = _f32arr(x), _f32arr(w)
        state = _f32arr(state, True)
        tokens, channels = x.shape
        out = np.empty_like(x)
        self._call("orc_conv_l2norm", _ptr(x), _ptr(state), _ptr(w), _ptr(out), tokens, channels, w.shape[1], l2_channels,
                   d, eps)
        return out

    def round_bf16(self, x):
        x = _f32arr(x, True)
        self._call("orc_round_bf16", _ptr(x), x.size)
        return x

    def round_fp16(self, x):
        x = _f32arr(x, True)
        self._call("orc_round_fp16", _ptr(x), x.size)
        return x


_cache: dict[str, Oracle] = {}


def load(kind: str = "port") -> Oracle:
    if kind in _cache:
        return _cache[kind]
    if kind == "port":
        if not PORT_LIB.exists():
            build(ref=False)
        o = Oracle(PORT_LIB)
    elif kind == "reference":
        if not REF_LIB.exists():
            raise FileNotFoundError(f"{REF_LIB} not built (needs the reference checkout: make -C oracle ref)")
        o = Oracle(REF_LIB, fallback=load("port"))
    else:
        raise ValueError(kind)
    _cache[kind] = o
    return o


def have_reference() -> bool:
    return REF_LIB.exists()


def best() -> Oracle:
    """The compiled reference when it is available, else the port."""
    return load("reference") if have_reference() else load("port")


# --- numpy helpers shared by the tests and the benchmark -------------------
def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even (src/kernels/core.hip:70-73)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    return bf16_to_f32(bf16_bits(x))
