"""ctypes binding of libhalo_b200.so: one Python callable per C-ABI entry point.

The signatures mirror include/halo_b200.h. There is no fallback of any kind:
if the shared library is missing, loading raises, and a failing call raises
HaloError with the library's own message.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libhalo_b200.so"

F32, F16, BF16 = 0, 1, 2

_p, _u32, _u64, _f, _i, _sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_float, C.c_int, C.c_size_t

# name -> argument types between `stream` and the trailing (err, errlen)
SIGNATURES: dict[str, list] = {
    "halo_b200_add": [_p, _p, _u32],
    "halo_b200_axpy": [_p, _p, _f, _u32],
    "halo_b200_rmsnorm": [_p, _p, _p, _u32, _f, _u32, _u32],
    "halo_b200_rmsnorm_rows": [_p, _p, _p, _u32, _f, _u32, _u32, _u32],
    "halo_b200_rmsnorm_rows_r16": [_p, _p, _p, _u32, _f, _u32, _u32, _u32],
    "halo_b200_rmsnorm_rows_rb": [_p, _p, _p, _u32, _f, _u32, _u32, _u32],
    "halo_b200_rmsnorm_rows_h": [_p, _i, _p, _p, _p, _u32, _f, _u32, _u32, _p, _p, _u32, _u32, _u32],
    "halo_b200_rmsnorm_y": [_p, _p, _u32, _f, _u32, _u32, _u32, _u32],
    "halo_b200_rmsnorm_ex": [_p, _i, _p, _p, _i, _u32, _f, _u32, _u32, _i, _u32],
    "halo_b200_add_rmsnorm": [_p, _p, _i, _p, _i, _p, _i, _p, _p, _p, _u32, _f, _u32],
    "halo_b200_quantize_q8_rows": [_p, _p, _p, _u32, _u32],
    "halo_b200_quantize_q8_kblocked": [_p, _p, _p, _u32, _u32],
    "halo_b200_q8x_cols": [_p, _u32, _u32, _p, _p, _p, _p, _u32],
    "halo_b200_hc_norm_q8x": [_p, _p, _p, _p, _u32, _u32, _p, _p, _p, _p, _u32],
    "halo_b200_encode_q8_0_rows": [_p, _i, _p, _u32, _u32],
    "halo_b200_l2norm": [_p, _u32, _f, _u32],
    "halo_b200_l2norm_ex": [_p, _i, _p, _i, _u32, _f, _u32],
    "halo_b200_gated_norm": [_p, _p, _p, _u32, _f, _u32, _u32],
    "halo_b200_gated_norm_h": [_p, _p, _p, _p, _u32, _f, _u32, _u32],
    "halo_b200_gated_norm_hz": [_p, _p, _p, _p, _u32, _f, _u32, _u32],
    "halo_b200_gated_norm_h128w": [_p, _p, _p, _p, _u32, _f, _u32],
    "halo_b200_gated_norm_h128w_hh": [_p, _p, _p, _p, _u32, _f, _u32],
    "halo_b200_gated_norm_ex": [_p, _i, _p, _p, _i, _p, _i, _u32, _f, _u32, _u32],
    "halo_b200_rope_neox": [_p, _u32, _u32, _u32, _f, _u32],
    "halo_b200_rope_neox_rows": [_p, _u32, _u32, _u32, _u32, _f, _u32],
    "halo_b200_rope_neox_p": [_p, _p, _u32, _u32, _u32, _u32, _f, _u32],
    "halo_b200_rope_neox_blocks": [_p, _u32, _u32, _u32, _u32, _f, _u32],
    "halo_b200_rope_neox_p_y": [_p, _p, _u32, _u32, _u32, _u32, _f, _u32, _u32, _u32, _u32],
    "halo_b200_rope_ex": [_p, _u32, _p, _u32, _i, _u32, _u32, _f, _u32, _p, _u32, _u32, _u32, _u32, _p],
    "halo_b200_split_qgate": [_p, _p, _p, _u32, _u32],
    "halo_b200_split_qgate_y": [_p, _p, _p, _u32, _u32, _u32, _u32, _u32],
    "halo_b200_split_qgate_norm_rope": [_p, _p, _p, _p, _f, _u32, _u32, _u32, _f, _u32, _u32],
    "halo_b200_norm_rope_rows": [_p, _p, _f, _u32, _u32, _u32, _u32, _f, _p, _u32],
    "halo_b200_norm_rope_ex": [_p, _i, _u64, _p, _i, _p, _p, _p, _i, _f, _u32, _u32, _u32, _u32, _f, _p, _u32, _u32,
                               _u32, _u32, _p],
    "halo_b200_norm_rope_qk_ex": [_p, _u64, _p, _p, _p, _u32, _p, _p, _p, _p, _u32, _i, _i, _i, _f, _u32, _u32, _u32, _f,
                                  _p, _u32, _u32, _u32, _u32, _p],
    "halo_b200_rope_table_ex": [_p, _u32, _u32, _f, _p, _u32, _u32, _u32, _u32, _p],
    "halo_b200_norm_rope_qk_table_ex": [_p, _u64, _p, _p, _p, _u32, _p, _p, _p, _p, _u32, _i, _i, _i, _f, _u32, _u32, _u32, _p],
    "halo_b200_norm_rope_qk_noalloc": [_p, _u64, _p, _p, _p, _u32, _p, _p, _p, _p, _u32, _i, _i, _i, _f, _u32, _u32, _u32, _f,
                                       _p, _u32, _u32, _u32, _u32, _p],
    "halo_b200_silu_mul": [_p, _p, _u32],
    "halo_b200_silu_mul_h": [_p, _p, _p, _u32],
    "halo_b200_silu_mul_ex": [_p, _p, _i, _p, _i, _u64],
    "halo_b200_silu_mul_multi_ex": [_u32, _p, _p, _p, _p, _i, _i],
    "halo_b200_sigmoid_gate": [_p, _p, _u32],
    "halo_b200_matvec_q8_0_embed": [_p, _p, _u32, _u32, _u64],
    "halo_b200_matvec_q8_0_embed_p": [_p, _p, _p, _u32, _u64],
    "halo_b200_matvec_q8_0_embed_rows": [_p, _p, _p, _u32, _u64, _u32],
    "halo_b200_hc_combine_norm_rows": [_p, _i, _p, _p, _p, _p, _p, _u32, _u32, _f, _p, _p, _u32, _p, _u32, _u32],
    "halo_b200_hc_combine_norm_rows_q8": [_p, _p, _p, _p, _p, _p, _u32, _u32, _f, _p, _p, _u32, _p, _u32, _p, _p, _u32],
    "halo_b200_hc_combine_norm_tok": [_p, _i, _p, _p, _p, _p, _u32, _f, _p, _p, _u32, _p, _u32, _u32],
    "halo_b200_hc_combine_norm_tok_moe": [_p, _i, _p, _p, _p, _p, _p, _u32, _p, _p, _p, _u32, _f, _p, _p, _u32, _p, _u32,
                                          _u32],
    "halo_b200_hc_combine_norm_ex": [_p, _i, _p, _i, _p, _p, _i, _p, _i, _p, _u32, _p, _p, _p, _u32, _p, _p, _u32, _u32, _f,
                                     _u32],
    "halo_b200_hc_combine_norm_moe_ex": [_p, _i, _p, _i, _p, _p, _p, _i, _p, _u32, _p, _p, _i, _p, _i, _p, _u32, _p, _p, _p,
                                         _u32, _u32, _u32, _f, _u32],
    "halo_b200_hc_combine_rows": [_p, _i, _p, _p, _u32, _u32, _u32],
    "halo_b200_hc_combine_rows_ex": [_p, _i, _p, _i, _p, _u32, _u32, _u32],
    "halo_b200_broadcast_rows": [_p, _i, _p, _u32, _u32, _u32],
    "halo_b200_broadcast_rows_ex": [_p, _i, _p, _i, _u32, _u32, _u32],
    "halo_b200_hc_mix_rows": [_p, _p, _p, _u32, _u32, _u32],
    "halo_b200_hc_mix_rows_ex": [_p, _p, _p, _i, _u32, _u32, _u32],
    "halo_b200_axpy_sigmoid_rows": [_p, _p, _p, _u32, _u32],
    "halo_b200_inject_reduce": [_p, _p, _u32, _u32, _u32],
    "halo_b200_res_to_f32": [_p, _p, _i, _u32],
    "halo_b200_hc_norm_scales": [_p, _p, _u32, _f, _u32],
    "halo_b200_conv_l2norm_prefill": [_p, _p, _p, _p, _u32, _u32, _u32, _f, _u32, _u32],
    "halo_b200_conv_l2norm_prefill8": [_p, _i, _p, _p, _p, _i, _u32, _u32, _u32, _f, _u32],
    "halo_b200_conv_l2norm_ex": [_p, _i, _p, _p, _p, _i, _u32, _u32, _u32, _u32, _f, _u32],
    "halo_b200_conv_state_advance": [_p, _i, _p, _u32, _u32, _u32],
    "halo_b200_conv_l2norm": [_p, _p, _p, _p, _u32, _u32, _u32, _f, _u32],
    "halo_b200_conv_l2norm_y": [_p, _p, _u32, _u32, _p, _p, _u32, _u32, _u32, _f, _u32, _u32, _u32],
    "halo_b200_conv_step": [_p, _p, _p, _p, _u32, _u32],
    "halo_b200_copy_at": [_p, _i, _p, _p, _u32, _u32, _u32],
    "halo_b200_copy_at_y": [_p, _u32, _u32, _i, _p, _p, _u32, _u32, _u32, _u32, _u32, _u32],
    "halo_b200_copy": [_p, _p, _u32],
    "halo_b200_f16_rows": [_p, _p, _u32],
    "halo_b200_scale_silu": [_p, _p, _i, _f, _u32],
    "halo_b200_moe_combine_grouped": [_p, _p, _p, _p, _u32, _u32, _u32],
    "halo_b200_moe_combine_shared": [_p, _p, _p, _p, _p, _p, _u32, _u32, _u32],
    "halo_b200_moe_combine": [_p, _p, _p, _u32, _u32],
    "halo_b200_axpy_slot": [_p, _p, _p, _u32, _u32],
    "halo_b200_moe_combine_ex": [_p, _i, _p, _p, _p, _i, _p, _p, _i, _u32, _u32, _u32],
    "halo_b200_embed_q8_0_ex": [_p, _u64, _u32, _p, _u32, _u32, _u32, _p, _i, _u32],
}

# Entry points with other calling shapes.
OTHER_EXPORTS = ["halo_b200_version", "halo_b200_launch", "halo_b200_kernel_count", "halo_b200_kernel_name",
                 "halo_b200_tune", "halo_b200_conv_stage_timeouts", "halo_b200_stage_timeouts"]


class HaloArgValue(C.Union):
    _fields_ = [("ptr", C.c_void_p), ("bytes", C.c_uint8 * 8)]


class HaloArg(C.Structure):
    """struct halo_b200_arg."""
    _fields_ = [("is_buffer", C.c_uint32), ("size", C.c_uint32), ("v", HaloArgValue)]


class HaloError(RuntimeError):
    pass


class Library:
    def __init__(self, path: Path = LIB_PATH):
        if not Path(path).exists():
            raise FileNotFoundError(
                f"{path} is missing: build it with `python -m halo_flash_b200.build` "
                "(the CUDA library is the only implementation; there is no CPU fallback)")
        self.path = Path(path)
        self.cdll = C.CDLL(str(path))
        self._fn = {}
        for name, mid in SIGNATURES.items():
            f = getattr(self.cdll, name)
            f.restype = C.c_int
            f.argtypes = [_p, *mid, C.c_char_p, _sz]
            self._fn[name] = f
        self.cdll.halo_b200_version.restype = C.c_char_p
        self.cdll.halo_b200_version.argtypes = []
        self.cdll.halo_b200_kernel_count.restype = _sz
        self.cdll.halo_b200_kernel_count.argtypes = []
        self.cdll.halo_b200_kernel_name.restype = C.c_char_p
        self.cdll.halo_b200_kernel_name.argtypes = [_sz]
        self.cdll.halo_b200_tune.restype = C.c_int
        self.cdll.halo_b200_tune.argtypes = [C.c_char_p, C.c_int]
        self.cdll.halo_b200_launch.restype = C.c_int
        self.cdll.halo_b200_launch.argtypes = [_p, C.c_char_p, C.POINTER(HaloArg), _sz, C.POINTER(C.c_uint32 * 3),
                                               C.POINTER(C.c_uint32 * 3), C.c_char_p, _sz]
        self.calls = 0  # kernel-launching calls made through this binding (for launch accounting)

    def version(self) -> str:
        return self.cdll.halo_b200_version().decode()

    def tune(self, key: str, value: int) -> None:
        if self.cdll.halo_b200_tune(key.encode(), value) != 0:
            raise HaloError(f"halo_b200_tune: bad key or value ({key}={value})")

    def kernel_names(self) -> list[str]:
        return [self.cdll.halo_b200_kernel_name(i).decode() for i in range(self.cdll.halo_b200_kernel_count())]

    def call(self, name: str, stream: int, *args) -> None:
        """Invoke `halo_b200_<name>`; raises HaloError with the library's message on failure."""
        err = C.create_string_buffer(512)
        rc = self._fn["halo_b200_" + name](stream, *args, err, len(err))
        self.calls += 1
        if rc != 0:
            raise HaloError(err.value.decode(errors="replace"))

    def launch(self, stream: int, name: str, args: list[HaloArg], grid, block) -> None:
        arr = (HaloArg * max(1, len(args)))(*args)
        g = (C.c_uint32 * 3)(*grid)
        b = (C.c_uint32 * 3)(*block)
        err = C.create_string_buffer(512)
        rc = self.cdll.halo_b200_launch(stream, name.encode(), arr, len(args), C.byref(g), C.byref(b), err, len(err))
        self.calls += 1
        if rc != 0:
            raise HaloError(err.value.decode(errors="replace"))


_lib: Library | None = None


def lib() -> Library:
    global _lib
    if _lib is None:
        _lib = Library()
    return _lib
