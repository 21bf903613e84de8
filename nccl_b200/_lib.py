"""Locates, builds and loads the native library (``libnccl_b200.so``) and declares its C API.

The library exports the NCCL host API (reference: src/nccl.h.in); everything in this package
reaches the data plane through these ctypes prototypes.
"""
import ctypes
import os
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
# NCCL_B200_LIBRARY points the package at another build of the library (e.g. one made with `make SAN=address`).
LIB_PATH = os.environ.get("NCCL_B200_LIBRARY") or os.path.join(_HERE, "lib", "libnccl_b200.so")

_lock = threading.Lock()
_lib = None

ncclResult_t = ctypes.c_int
ncclComm_t = ctypes.c_void_p
cudaStream_t = ctypes.c_void_p


class ncclUniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_char * 128)]


class ncclConfig_t(ctypes.Structure):
    _fields_ = [
        ("size", ctypes.c_size_t), ("magic", ctypes.c_uint), ("version", ctypes.c_uint),
        ("blocking", ctypes.c_int), ("cgaClusterSize", ctypes.c_int), ("minCTAs", ctypes.c_int),
        ("maxCTAs", ctypes.c_int), ("netName", ctypes.c_char_p), ("splitShare", ctypes.c_int),
        ("trafficClass", ctypes.c_int), ("commName", ctypes.c_char_p), ("collnetEnable", ctypes.c_int),
        ("CTAPolicy", ctypes.c_int), ("shrinkShare", ctypes.c_int), ("nvlsCTAs", ctypes.c_int),
        ("nChannelsPerNetPeer", ctypes.c_int), ("nvlinkCentricSched", ctypes.c_int),
        ("graphUsageMode", ctypes.c_int), ("numRmaCtx", ctypes.c_int), ("maxP2pPeers", ctypes.c_int),
        ("graphStreamOrdering", ctypes.c_int),
    ]


class ncclSimInfo_t(ctypes.Structure):
    _fields_ = [("size", ctypes.c_size_t), ("magic", ctypes.c_uint), ("version", ctypes.c_uint),
                ("estimatedTime", ctypes.c_float)]


UNDEF_INT = -2147483648
NCCL_VERSION_CODE = 23007


def make_config(**kw):
    """An ncclConfig_t initialised like NCCL_CONFIG_INITIALIZER, with keyword overrides."""
    c = ncclConfig_t()
    c.size = ctypes.sizeof(ncclConfig_t)
    c.magic = 0xCAFEBEEF
    c.version = NCCL_VERSION_CODE
    for name, typ in ncclConfig_t._fields_[3:]:
        setattr(c, name, None if typ is ctypes.c_char_p else UNDEF_INT)
    for k, v in kw.items():
        setattr(c, k, v.encode() if isinstance(v, str) else v)
    return c


def build(jobs=None, verbose=False):
    """Compiles the native library in-tree with make (nvcc for sm_100a)."""
    jobs = jobs or os.cpu_count() or 4
    cmd = ["make", "-C", _ROOT, "-j%d" % jobs]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout[-8000:])
    if res.returncode != 0:
        raise RuntimeError("building libnccl_b200.so failed")
    return LIB_PATH


_PROTOS = {
    "ncclGetVersion": [ctypes.POINTER(ctypes.c_int)],
    "ncclGetUniqueId": [ctypes.POINTER(ncclUniqueId)],
    "ncclCommInitRank": [ctypes.POINTER(ncclComm_t), ctypes.c_int, ncclUniqueId, ctypes.c_int],
    "ncclCommInitRankConfig": [ctypes.POINTER(ncclComm_t), ctypes.c_int, ncclUniqueId, ctypes.c_int, ctypes.POINTER(ncclConfig_t)],
    "ncclCommInitRankScalable": [ctypes.POINTER(ncclComm_t), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ncclUniqueId), ctypes.POINTER(ncclConfig_t)],
    "ncclCommInitAll": [ctypes.POINTER(ncclComm_t), ctypes.c_int, ctypes.POINTER(ctypes.c_int)],
    "ncclCommFinalize": [ncclComm_t],
    "ncclCommDestroy": [ncclComm_t],
    "ncclCommAbort": [ncclComm_t],
    "ncclCommRevoke": [ncclComm_t, ctypes.c_int],
    "ncclCommSplit": [ncclComm_t, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ncclComm_t), ctypes.POINTER(ncclConfig_t)],
    "ncclCommShrink": [ncclComm_t, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.POINTER(ncclComm_t), ctypes.POINTER(ncclConfig_t), ctypes.c_int],
    "ncclCommGetUniqueId": [ncclComm_t, ctypes.POINTER(ncclUniqueId)],
    "ncclCommGrow": [ncclComm_t, ctypes.c_int, ctypes.POINTER(ncclUniqueId), ctypes.c_int, ctypes.POINTER(ncclComm_t), ctypes.POINTER(ncclConfig_t)],
    "ncclCommGetAsyncError": [ncclComm_t, ctypes.POINTER(ctypes.c_int)],
    "ncclCommCount": [ncclComm_t, ctypes.POINTER(ctypes.c_int)],
    "ncclCommCuDevice": [ncclComm_t, ctypes.POINTER(ctypes.c_int)],
    "ncclCommUserRank": [ncclComm_t, ctypes.POINTER(ctypes.c_int)],
    "ncclCommRegister": [ncclComm_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)],
    "ncclCommDeregister": [ncclComm_t, ctypes.c_void_p],
    "ncclCommWindowRegister": [ncclComm_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int],
    "ncclCommWindowDeregister": [ncclComm_t, ctypes.c_void_p],
    "ncclWinGetUserPtr": [ncclComm_t, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)],
    "ncclCommSuspend": [ncclComm_t, ctypes.c_int],
    "ncclCommResume": [ncclComm_t],
    "ncclCommMemStats": [ncclComm_t, ctypes.c_int, ctypes.POINTER(ctypes.c_uint64)],
    "ncclMemAlloc": [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t],
    "ncclMemFree": [ctypes.c_void_p],
    "ncclRedOpCreatePreMulSum": [ctypes.POINTER(ctypes.c_int), ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ncclComm_t],
    "ncclRedOpDestroy": [ctypes.c_int, ncclComm_t],
    "ncclAllReduce": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclReduce": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclBroadcast": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclBcast": [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclReduceScatter": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclAllGather": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclAlltoAll": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclGather": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclScatter": [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclSend": [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclRecv": [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t],
    "ncclSignal": [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint, ncclComm_t, cudaStream_t],
    "ncclGroupStart": [],
    "ncclGroupEnd": [],
    "ncclGroupSimulateEnd": [ctypes.POINTER(ncclSimInfo_t)],
}


def declare(lib):
    """Attaches argtypes/restype of the NCCL C API to a loaded library (ours or the reference's)."""
    for name, args in _PROTOS.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = ncclResult_t
    for name in ("ncclGetErrorString",):
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = [ctypes.c_int]
            fn.restype = ctypes.c_char_p
    fn = getattr(lib, "ncclGetLastError", None)
    if fn is not None:
        fn.argtypes = [ncclComm_t]
        fn.restype = ctypes.c_char_p
    return lib


def load(path=None):
    """Loads the native library (building it first when the .so is missing)."""
    global _lib
    if path is not None:
        return declare(ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL))
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                build()
            _lib = declare(ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL))
        return _lib


class NcclError(RuntimeError):
    def __init__(self, code, what, detail=""):
        self.code = code
        super().__init__("%s failed: %s%s" % (what, ERROR_NAMES.get(code, str(code)), (" (" + detail + ")") if detail else ""))


ERROR_NAMES = {0: "ncclSuccess", 1: "ncclUnhandledCudaError", 2: "ncclSystemError", 3: "ncclInternalError",
               4: "ncclInvalidArgument", 5: "ncclInvalidUsage", 6: "ncclRemoteError", 7: "ncclInProgress", 8: "ncclTimeout"}


def check(code, what, lib=None):
    if code != 0 and code != 7:
        detail = ""
        try:
            detail = (lib or load()).ncclGetLastError(None).decode(errors="replace")
        except Exception:
            pass
        raise NcclError(code, what, detail)
    return code
