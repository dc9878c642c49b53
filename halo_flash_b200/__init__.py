"""halo_flash_b200: B200 (sm_100a) CUDA kernels for halo-flash's fused per-layer
elementwise path, behind the C ABI declared in include/halo_b200.h.

    csrc/      the kernels and the C ABI (built in-tree into libhalo_b200.so)
    _lib.py    ctypes binding of every entry point
    ops.py     the five op groups on torch CUDA tensors
    device.py  a CUDA stand-in for the reference's rt::Device (launch by kernel name)
    chain.py   the per-layer op chain (36 DeltaNet + 12 GQA layers) and its token sharding

The CUDA library is the only implementation: importing works anywhere, but every
op raises unless libhalo_b200.so is built and a CUDA device is present.
"""
from ._lib import BF16, F16, F32, HaloError, lib  # noqa: F401

__all__ = ["lib", "HaloError", "F32", "F16", "BF16"]
