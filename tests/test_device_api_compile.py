"""The device API headers accept kernels written with the reference's spellings (team tags, scoped barrier
sessions with memory orders, typed put / signal actions, team arithmetic): compile-only, no GPU needed."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_spelling_compiles(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is not installed")
    src = os.path.join(ROOT, "tests", "data", "device_api_reference_spelling.cu")
    p = subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + os.path.join(ROOT, "include"),
                        "-diag-suppress", "550", "-c", src, "-o", str(tmp_path / "out.o")], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr


def test_device_utility_helpers_compile_and_divide_exactly(tmp_path):
    """Fast division, rolling comparisons and pointer helpers: the kernel only has to compile; the reciprocal
    arithmetic behind ncclFastDiv32 is replayed on the host for divisors and dividends around every boundary."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is not installed")
    src = os.path.join(ROOT, "tests", "data", "device_utility_check.cu")
    exe = str(tmp_path / "utility_check")
    p = subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I" + os.path.join(ROOT, "include"),
                        "-cudart", "static", src, "-o", exe], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    assert subprocess.run([exe]).returncode == 0
