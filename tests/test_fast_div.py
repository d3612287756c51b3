"""CPU test of the multiply-shift division the HBM-bound gather kernels use in place of hardware divisions
(csrc/fast_div.cuh): the host side of the same header, compiled by nvcc, checked against x / d and x % d."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fast_div_is_exact_below_2_to_31(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    exe = str(tmp_path / "fast_div_check")
    src = os.path.join(ROOT, "tests", "fast_div_check.cu")
    subprocess.run([nvcc, "-O2", "-std=c++17", "-o", exe, src], check=True, capture_output=True, timeout=300)
    out = subprocess.run([exe, "5000"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert " 0 wrong" in out.stdout, out.stdout
