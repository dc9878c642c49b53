"""The C++ backend of the reference's device interface (halo_flash_b200/rt/cuda_device.cpp), driven by a
C++ program written against halo::rt::Device alone and checked against the reference's own CPU operators
(tests/cpp/rt_device_check.cpp). The program is built where the reference checkout is present (its headers
are needed) and travels as a binary; this test runs it (GPU only)."""
import os
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "halo_flash_b200" / "rt" / "_build" / "rt_device_check"


def test_reference_device_interface_drives_the_kernels():
    if not BIN.exists():
        pytest.skip("rt_device_check is built only where the reference checkout is present (make -C halo_flash_b200/rt)")
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = f"{ROOT / 'halo_flash_b200'}:/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    p = subprocess.run([str(BIN)], capture_output=True, text=True, timeout=120, env=env)
    print(p.stdout, p.stderr)
    assert p.returncode == 0 and "ALL PASS" in p.stdout, p.stdout + p.stderr
    assert p.stdout.count("PASS") >= 6
