"""A CUDA stand-in for the reference's device layer, for hosts that drive the
kernels the way halo-flash's engine does.

Mirrors `halo::rt::Device` (src/rt/device.hpp:77-137): buffers are allocated,
uploaded and downloaded through the device; kernels are looked up by name and
launched with a grid, a block and an ordered list of `Arg.Buf` / `Arg.Val`
arguments (src/rt/device.hpp:35-59); launches between begin_capture and
end_capture are recorded into a replayable graph whose arguments are frozen
(device.hpp:66-75). Errors are raised as exceptions instead of the C++
`bool + std::string* error` pair. Method names are the reference's in
snake_case.

The device owns one non-blocking stream, like the HIP backend
(src/rt/hip_device.cpp:49-50). Kernel launches go to `halo_b200_launch`, which
decodes row counts from the grid as the reference kernels read blockIdx.
"""
from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass, field

import numpy as np
import torch

from ._lib import HaloArg, HaloError, lib


@dataclass
class Buffer:
    """Device memory: `device` is the address kernels see (rt::Buffer)."""
    tensor: torch.Tensor | None = None
    bytes: int = 0

    @property
    def device(self) -> int:
        return 0 if self.tensor is None else self.tensor.data_ptr()

    def __bool__(self) -> bool:
        return self.tensor is not None


@dataclass
class Arg:
    """One launch argument (rt::Arg): a buffer (+ byte offset) or a by-value scalar of <= 8 bytes."""
    is_buffer: bool
    buffer: Buffer | None = None
    offset: int = 0
    raw: bytes = b""

    @staticmethod
    def Buf(b: Buffer, offset_bytes: int = 0) -> "Arg":
        return Arg(True, b, offset_bytes)

    @staticmethod
    def U32(v: int) -> "Arg":
        return Arg(False, raw=struct.pack("<I", v & 0xFFFFFFFF))

    @staticmethod
    def U64(v: int) -> "Arg":
        return Arg(False, raw=struct.pack("<Q", v))

    @staticmethod
    def F32(v: float) -> "Arg":
        return Arg(False, raw=struct.pack("<f", v))

    Null = None  # set below: a null optional pointer, passed as Arg::Val<uint64_t>(0)

    def to_c(self) -> HaloArg:
        a = HaloArg()
        if self.is_buffer:
            a.is_buffer = 1
            a.size = 8
            a.v.ptr = self.buffer.device + self.offset
        else:
            a.is_buffer = 0
            a.size = len(self.raw)
            for i, byte in enumerate(self.raw):
                a.v.bytes[i] = byte
        return a


Arg.Null = Arg.U64(0)


@dataclass
class Graph:
    exec: torch.cuda.CUDAGraph | None = None

    def __bool__(self) -> bool:
        return self.exec is not None


@dataclass
class Device:
    index: int = 0
    _names: list[str] = field(default_factory=list)
    _capturing: torch.cuda.CUDAGraph | None = None
    _capture_ctx: object = None

    @staticmethod
    def create(index: int = 0) -> "Device":
        if not torch.cuda.is_available():
            raise HaloError("no CUDA device: halo_flash_b200 has no CPU path")
        d = Device(index)
        d._torch_device = torch.device("cuda", index)
        d.stream = torch.cuda.Stream(device=d._torch_device)
        d._names = lib().kernel_names()
        return d

    # ---- memory -----------------------------------------------------------
    def alloc(self, nbytes: int) -> Buffer:
        return Buffer(torch.empty(max(nbytes, 1), dtype=torch.uint8, device=self._torch_device), nbytes)

    def free(self, b: Buffer) -> None:
        b.tensor, b.bytes = None, 0

    def upload(self, dst: Buffer, offset: int, src) -> None:
        if self._capturing is not None:
            raise HaloError("upload inside a capture")
        host = torch.from_numpy(np.frombuffer(np.ascontiguousarray(src).tobytes(), dtype=np.uint8).copy())
        if offset + host.numel() > dst.bytes:
            raise HaloError("upload past the end of the buffer")
        with torch.cuda.stream(self.stream):
            dst.tensor[offset:offset + host.numel()].copy_(host)
        self.stream.synchronize()

    def download(self, src: Buffer, offset: int, nbytes: int, dtype=np.uint8) -> np.ndarray:
        if self._capturing is not None:
            raise HaloError("download inside a capture")
        if offset + nbytes > src.bytes:
            raise HaloError("download past the end of the buffer")
        with torch.cuda.stream(self.stream):
            host = src.tensor[offset:offset + nbytes].cpu()
        self.stream.synchronize()
        return host.numpy().view(dtype).copy()

    def fill(self, dst: Buffer, value: int) -> None:
        with torch.cuda.stream(self.stream):
            dst.tensor.fill_(value)

    # ---- kernels ----------------------------------------------------------
    def kernel(self, name: str) -> int:
        """KernelId of a kernel this library replaces; raises for any other name."""
        try:
            return self._names.index(name)
        except ValueError:
            raise HaloError(f"kernel {name} is not part of the layer-op path") from None

    def launch(self, kernel: int, grid, block, args: list[Arg]) -> None:
        g = tuple(grid) + (1,) * (3 - len(grid))
        b = tuple(block) + (1,) * (3 - len(block))
        with torch.cuda.device(self.index):  # the launch goes to the CURRENT device: make it this object's
            lib().launch(self.stream.cuda_stream, self._names[kernel], [a.to_c() for a in args], g, b)

    def synchronize(self) -> None:
        if self._capturing is not None:
            raise HaloError("synchronize inside a capture")
        self.stream.synchronize()

    # ---- graphs -----------------------------------------------------------
    def begin_capture(self) -> None:
        if self._capturing is not None:
            raise HaloError("capture already in progress")
        self._capturing = torch.cuda.CUDAGraph()
        self._capture_ctx = torch.cuda.graph(self._capturing, stream=self.stream)
        self._capture_ctx.__enter__()

    def end_capture(self) -> Graph:
        if self._capturing is None:
            raise HaloError("no capture in progress")
        self._capture_ctx.__exit__(None, None, None)
        g, self._capturing, self._capture_ctx = Graph(self._capturing), None, None
        return g

    def launch_graph(self, graph: Graph) -> None:
        with torch.cuda.stream(self.stream):
            graph.exec.replay()

    def free_graph(self, graph: Graph) -> None:
        graph.exec = None
