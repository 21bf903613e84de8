"""Versions of the package and of the native library it loads, as a record and as a printed summary.

Reference parity: bindings/nccl4py/nccl/_show_versions.py (LibraryInfo, VersionInfo, get_version, show_versions).
"""
import ctypes
import pathlib
from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class LibraryInfo:
    version: Tuple[int, int, int]
    cuda_variant: Optional[Tuple[int, int]]   # CUDA toolkit the library was built with
    path: Optional[pathlib.Path]
    build: Optional[str] = None               # source revision stamped into the library

    def __str__(self):
        out = "%d.%d.%d" % self.version
        if self.cuda_variant is not None:
            out += "+cuda%d.%d" % self.cuda_variant
        if self.build:
            out += " (%s)" % self.build
        if self.path is not None:
            out += " @ %s" % self.path
        return out


@dataclass(frozen=True)
class VersionInfo:
    nccl4py: str
    nccl: Optional[LibraryInfo]
    nccl_ep: Optional[LibraryInfo]


def _package_version():
    try:
        from importlib.metadata import version
        return version("nccl_b200")
    except Exception:
        return "0+in-tree"


def get_version():
    nccl = nccl_ep = None
    try:
        from .. import _lib
        lib = _lib.load()
        v = ctypes.c_int(0)
        lib.ncclGetVersion(ctypes.byref(v))
        code = v.value
        cuda = None
        lib.b200CudaBuildVersion.restype = ctypes.c_int
        cv = lib.b200CudaBuildVersion()   # CUDART_VERSION of the toolkit that compiled the library
        if cv > 0:
            cuda = (cv // 1000, (cv % 1000) // 10)
        lib.b200GitVersion.restype = ctypes.c_char_p
        build = (lib.b200GitVersion() or b"").decode() or None
        path = pathlib.Path(lib._name)
        nccl = LibraryInfo((code // 10000, (code % 10000) // 100, code % 100), cuda, path, build)
        ev = ctypes.c_int(0)
        if lib.ncclEpGetVersion(ctypes.byref(ev)) == 0:
            nccl_ep = LibraryInfo((ev.value // 10000, (ev.value % 10000) // 100, ev.value % 100), cuda, path, build)
    except (OSError, AttributeError, RuntimeError):
        pass
    return VersionInfo(nccl4py=_package_version(), nccl=nccl, nccl_ep=nccl_ep)


def show_versions():
    v = get_version()
    print()
    print("NCCL versions")
    print("-------------")
    print("%-12s: %s" % ("nccl4py", v.nccl4py))
    print("%-12s: %s" % ("libnccl", v.nccl if v.nccl is not None else "not available"))
    print("%-12s: %s" % ("libnccl_ep", v.nccl_ep if v.nccl_ep is not None else "not available (same library)" if v.nccl else "not available"))
