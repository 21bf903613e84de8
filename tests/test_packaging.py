"""Distribution packages: the relocatable tarball and the Python wheel are built from the tree and carry the library,
the headers, the tools and the plugins. CPU only."""
import os
import shutil
import subprocess
import sys
import tarfile
import zipfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "nccl_b200", "lib", "libnccl_b200.so")


@pytest.mark.skipif(not os.path.exists(LIB), reason="the library is not built")
def test_tarball_has_library_headers_tools_and_plugins(tmp_path):
    if not shutil.which("xz"):
        pytest.skip("xz is not installed")
    p = subprocess.run(["make", "-C", os.path.join(ROOT, "pkg"), "txz", "OUT=" + str(tmp_path)], capture_output=True, text=True, timeout=1200)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    tars = [f for f in os.listdir(tmp_path) if f.endswith(".txz")]
    assert len(tars) == 1
    with tarfile.open(os.path.join(tmp_path, tars[0])) as t:
        names = set(n.split("/", 1)[1] for n in t.getnames() if "/" in n)
    for want in ("lib/libnccl_b200.so", "lib/libnccl_device_c.a", "include/nccl.h", "include/nccl_device.h", "include/nccl_device_c.h",
                 "include/nccl_device/core.h", "include/plugin/nccl_net.h", "bin/ncclparam", "bin/ncclras", "lib/pkgconfig/nccl_b200.pc",
                 "lib/nccl_b200/plugins/net/unix_net.so", "lib/nccl_b200/plugins/profiler/inspector.so"):
        assert want in names, want


@pytest.mark.skipif(not os.path.exists(LIB), reason="the library is not built")
def test_wheel_carries_the_native_library(tmp_path):
    p = subprocess.run(["make", "-C", os.path.join(ROOT, "pkg"), "wheel", "OUT=" + str(tmp_path), "PYTHON=" + sys.executable], capture_output=True, text=True, timeout=1200)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    wheels = [f for f in os.listdir(tmp_path) if f.endswith(".whl")]
    assert len(wheels) == 1 and "none-any" not in wheels[0], wheels   # platform wheel: it holds a shared library
    names = set(zipfile.ZipFile(os.path.join(tmp_path, wheels[0])).namelist())
    for want in ("nccl_b200/__init__.py", "nccl_b200/core.py", "nccl_b200/ops/ep.py", "nccl_b200/nccl4py/core/__init__.py", "nccl_b200/nccl4py/core/interop/torch.py", "nccl_b200/nccl4py/ep.py", "nccl_b200/lib/libnccl_b200.so",
                 "nccl_b200/lib/plugins/tuner/csv_tuner.so", "nccl_b200/bin/ncclparam", "nccl_b200/include/nccl.h", "nccl_b200/include/nccl_device/core.h"):
        assert want in names, want
    assert not os.path.exists(os.path.join(ROOT, "nccl_b200.egg-info"))


def test_every_example_program_is_built():
    """`make` turns every examples/*.cu into a program under nccl_b200/bin/examples (they run in the GPU suite)."""
    src = sorted(f[:-3] for f in os.listdir(os.path.join(ROOT, "examples")) if f.endswith(".cu"))
    built = set(os.listdir(os.path.join(ROOT, "nccl_b200", "bin", "examples")))
    assert src and not [s for s in src if s not in built]
