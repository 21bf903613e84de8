"""Wheel of the Python package with the native library inside (nccl_b200/lib, nccl_b200/bin) and the C headers
(nccl_b200/include), so that `pip install` of the wheel gives both the Python API and what C programs need.
The native parts are built by `make` first (run here when the library is missing).
Reference parity: pkg/python_wheel."""
import glob
import os
import shutil
import subprocess

from setuptools import setup
from setuptools.command.build_py import build_py
from setuptools.dist import Distribution

HERE = os.path.dirname(os.path.abspath(__file__))


class BinaryDistribution(Distribution):
    def has_ext_modules(self):   # the wheel carries a shared library: platform-specific tag
        return True


class BuildWithNative(build_py):
    def run(self):
        if not os.path.exists(os.path.join(HERE, "nccl_b200", "lib", "libnccl_b200.so")):
            subprocess.check_call(["make", "-j", str(os.cpu_count() or 4)], cwd=HERE)
        super().run()
        # headers travel inside the package
        dst = os.path.join(self.build_lib, "nccl_b200", "include")
        shutil.rmtree(dst, ignore_errors=True)
        shutil.copytree(os.path.join(HERE, "include"), dst)
        shutil.copy(os.path.join(HERE, "bindings", "ir", "nccl_device_c.h"), dst)


def native_files():
    out = []
    for pat in ("lib/*.so", "lib/*.a", "lib/plugins/*/*.so", "bin/ncclparam", "bin/ncclras"):
        out += [os.path.relpath(p, os.path.join(HERE, "nccl_b200")) for p in glob.glob(os.path.join(HERE, "nccl_b200", pat))]
    return out


setup(
    name="nccl_b200",
    version="2.30.7",
    description="Collective communication library for B200 GPUs with the NCCL host API, and its Python bindings",
    packages=["nccl_b200", "nccl_b200.ops", "nccl_b200.parallel", "nccl_b200.models", "nccl_b200.utils", "nccl_b200.nccl4py", "nccl_b200.nccl4py.core",
              "nccl_b200.nccl4py.core.interop"],
    package_data={"nccl_b200": native_files()},
    python_requires=">=3.9",
    cmdclass={"build_py": BuildWithNative},
    distclass=BinaryDistribution,
)
