"""The C-ABI surface, checked without a GPU: the library loads, exports every symbol
include/halo_b200.h declares, binds every one of them in Python, and rejects bad
arguments with -1 and a message before any launch is attempted."""
import ctypes as C
import re
from pathlib import Path

import pytest

from halo_flash_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "halo_b200.h").read_text()


def declared():
    names = set(re.findall(r"\b(halo_b200_[a-z0-9_]+)\s*\(", HEADER))
    assert len(names) >= 45
    return sorted(names)


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    for name in declared():
        assert hasattr(lib.cdll, name), f"{name} declared in halo_b200.h but not exported"
    assert lib.version().startswith("halo_b200")


def test_python_binding_covers_the_header():
    bound = set(_lib.SIGNATURES) | set(_lib.OTHER_EXPORTS)
    assert bound == set(declared())


def test_every_entry_point_cites_the_reference():
    """Each declaration sits under a comment naming the reference kernel it replaces, or saying
    outright that the reference has no counterpart."""
    for m in re.finditer(r"/\*(?:[^*]|\*(?!/))*\*/\s*((?:int|size_t|const char\*) halo_b200_[a-z0-9_]+\([^;]*;\s*)+", HEADER):
        comment = m.group(0)
        assert "src/" in comment or "No counterpart in the reference" in comment or "halo_b200_launch" in comment or "Version" in comment or "Names" in comment \
            or "Typed" in comment or "Tuning" in comment, comment[:120]


def test_kernel_names_are_reference_names():
    names = _lib.lib().kernel_names()
    assert len(names) == len(set(names)) >= 30
    for expect in ("halo_rmsnorm", "halo_rmsnorm_rows_rb", "halo_l2norm", "halo_gated_norm_h128w",
                   "halo_rope_neox_rows", "halo_rope_neox_p_y", "halo_split_qgate_norm_rope", "halo_norm_rope_rows",
                   "halo_silu_mul", "halo_silu_mul_h", "halo_quantize_q8_rows", "halo_matvec_q8_0_embed_rows"):
        assert expect in names


def _err_call(name, *args):
    with pytest.raises(_lib.HaloError) as e:
        _lib.lib().call(name, None, *args)
    return str(e.value)


def test_bad_arguments_are_rejected_with_a_message():
    assert "null" in _err_call("silu_mul", None, None, 8)
    assert "null" in _err_call("gated_norm", None, None, None, 128, 1e-6, 0, 4)
    assert "mode" in _err_call("gated_norm", 256, 256, 256, 128, 1e-6, 2, 4)
    assert "dtype" in _err_call("rmsnorm_ex", 256, 7, 256, 256, 0, 64, 1e-6, 0, 1, 0, 4)
    assert "% 32" in _err_call("add_rmsnorm", 256, 512, 0, 256, 1, None, 0, 1024, None, None, 48, 1e-6, 2)
    assert "xq and xd" in _err_call("add_rmsnorm", 256, 512, 0, 256, 1, None, 0, None, 1024, None, 64, 1e-6, 2)
    assert "rotary_dim" in _err_call("rope_neox", 256, 64, 66, 0, 1e7, 4)
    assert "rotary_dim" in _err_call("rope_neox", 256, 64, 15, 0, 1e7, 4)
    assert "cols % 32" in _err_call("matvec_q8_0_embed", 256, 256, 0, 48, 51)
    assert "row_bytes" in _err_call("matvec_q8_0_embed", 256, 256, 0, 64, 34)
    assert "iw needs gamma rows" in _err_call("rmsnorm_rows_h", 256, 0, 256, 256, 256, 64, 1e-6, 0, 2, 256, 256, 1, 0, 4)
    assert "inject goes with" in _err_call("hc_combine_norm_ex", 256, 0, 256, 0, None, 256, 0, 256, 0, None, 0, None, None,
                                           None, 0, None, None, 4, 64, 1e-6, 2)
    assert "hc rows per token" in _err_call("hc_combine_norm_rows", 256, 0, 256, 256, 256, 256, None, 4, 64, 1e-6, None,
                                            None, 0, None, 0, 7)
    assert "aligned" in _err_call("silu_mul", 258, 256, 8)  # fp32 pointer off by 2 bytes
    assert "1..256" in _err_call("norm_rope_rows", 256, 256, 1e-6, 512, 64, 0, 2, 1e7, None, 4)


def test_launch_by_name_rejects_unknown_and_malformed_calls():
    lib = _lib.lib()
    with pytest.raises(_lib.HaloError, match="unknown kernel"):
        lib.launch(None, "halo_gemv_q8r", [], (1, 1, 1), (256, 1, 1))
    a = _lib.HaloArg()
    a.is_buffer, a.v.ptr = 1, 256
    with pytest.raises(_lib.HaloError, match="argument list"):
        lib.launch(None, "halo_l2norm", [a], (4, 1, 1), (128, 1, 1))  # missing d, eps


def test_tune_keys_match_the_header():
    """Every key the header documents for halo_b200_tune is accepted (with 0, which every key allows, and which is then
    put back to its documented default), and an unknown key or value is refused. Host-only: no device is touched."""
    lib = _lib.lib()
    doc = HEADER[HEADER.index("Tuning hook for experiments"):HEADER.index("int halo_b200_tune")]
    keys = re.findall(r'"([a-z0-9_]+)"', doc)
    assert len(keys) >= 15 and len(set(keys)) == len(keys)
    defaults_on = set(re.findall(r'"([a-z0-9_]+)" \(1, the default', doc))
    assert {"pdl", "l2_keep", "rope_staged", "conv_staged", "embed_direct"} <= defaults_on
    for key in keys:
        lib.tune(key, 0)
        if key in defaults_on:
            lib.tune(key, 1)
    with pytest.raises(_lib.HaloError):
        lib.tune("no_such_key", 1)
    with pytest.raises(_lib.HaloError):
        lib.tune("pdl", 7)


def test_zero_sized_calls_succeed_without_a_device():
    """rows == 0 / n == 0 is a no-op (an empty prefill chunk), not an error."""
    lib = _lib.lib()
    lib.call("silu_mul", None, 256, 256, 0)
    lib.call("l2norm", None, 256, 128, 1e-6, 0)
    lib.call("rmsnorm_rows", None, 256, 256, 256, 64, 1e-6, 0, 1, 0)
    lib.call("matvec_q8_0_embed_rows", None, 256, 256, 256, 64, 68, 0)


def test_ops_reject_cpu_tensors():
    import torch
    from halo_flash_b200 import ops
    with pytest.raises(TypeError, match="CUDA tensor"):
        ops.silu_mul(torch.zeros(8), torch.zeros(8))
