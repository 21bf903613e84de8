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


def test_c_symbol_bindings_link_with_lto(tmp_path):
    """The device API delivered as C symbols with link-time-optimisation IR: a kernel that declares nothing but
    those symbols compiles to IR, and the device link against the library resolves every call for sm_100a."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is not installed")
    inc = ["-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(ROOT, "bindings", "ir")]
    lib = os.path.join(ROOT, "nccl_b200", "lib", "libnccl_device_c.a")
    if not os.path.exists(lib):
        os.makedirs(tmp_path / "o", exist_ok=True)
        obj = str(tmp_path / "o" / "nccl_device_c.o")
        p = subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=lto_100a", "-dc", *inc,
                            os.path.join(ROOT, "bindings", "ir", "nccl_device_c.cu"), "-o", obj], capture_output=True, text=True, timeout=300)
        assert p.returncode == 0, p.stdout + p.stderr
        lib = obj
    kobj = str(tmp_path / "kernel.o")
    p = subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=lto_100a", "-dc", *inc,
                        os.path.join(ROOT, "tests", "data", "ir_binding_kernel.cu"), "-o", kobj], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    p = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-dlto", "-cudart", "static", kobj, lib, "-o", str(tmp_path / "ir_kernel")],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    # an unresolved C symbol must fail the link (the check above is not vacuous)
    p = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-dlto", "-cudart", "static", kobj, "-o", str(tmp_path / "bad")],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode != 0
