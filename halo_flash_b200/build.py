"""Builds libhalo_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m halo_flash_b200.build [--force] [--verbose]

Objects go to halo_flash_b200/csrc/build/, the library to halo_flash_b200/libhalo_b200.so.
A source is recompiled when it or any header is newer than its object.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
LIB = PKG / "libhalo_b200.so"
INCLUDE = PKG.parent / "include"

SOURCES = ["norm.cu", "norm_odd.cu", "rope.cu", "elementwise.cu", "embed.cu", "quant.cu", "hc.cu", "conv.cu", "api.cu", "launch.cu", "static_scratch.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",  # multiplies and adds round separately, as the CPU operators do
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: libhalo_b200.so cannot be built (there is no CPU fallback)")


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted(INCLUDE.glob("*.h")) + [Path(__file__)]

    def compile_one(name: str):
        src, obj = CSRC / name, OBJ / (Path(name).stem + ".o")
        if not force and not _stale(obj, [src, *headers]):
            return name, None
        # HALO_B200_NVCC_FLAGS: extra flags for experiments (e.g. -DHALO_PF_HC=0); use --force when it changes
        extra = os.environ.get("HALO_B200_NVCC_FLAGS", "").split()
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name}:\n{p.stdout}\n{p.stderr}")
        (OBJ / (Path(name).stem + ".ptxas.txt")).write_text(p.stderr)
        return name, p.stderr

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as ex:
        results = list(ex.map(compile_one, SOURCES))
    rebuilt = [n for n, log in results if log is not None]
    if verbose:
        for n, log in results:
            if log:
                spills = [l for l in log.splitlines() if "spill" in l and "0 bytes spill stores" not in l]
                print(f"[build] {n}: compiled, {len(spills)} kernels with spills")
    objs = [OBJ / (Path(n).stem + ".o") for n in SOURCES]
    if force or rebuilt or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs)]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"link failed:\n{p.stdout}\n{p.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
