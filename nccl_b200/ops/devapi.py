"""Device API from Python: device communicators and the kernels built on the public device headers.

    dc  = DeviceComm(comm, barriers=64, ll_blocks=4, ll_slots=256)
    buf = dc.symmetric(numel, torch.bfloat16)           # tensor over a registered symmetric window
    dc.all_reduce(buf_in, buf_out, multimem=False)      # kernel written with nccl_device.h only
    dc.ar_rmsnorm(partial, residual, out, weight, eps)  # all-reduce + residual add + RMSNorm, one kernel

Reference parity: ncclDevCommCreate / ncclDevCommDestroy (src/include/nccl_device/core.h:152-175),
examples/06_device_api, contrib/nccl_ubx fused all-reduce + RMSNorm.
"""
import ctypes

from .. import _lib
from ..core import mem_alloc, mem_free
from ..utils.perf import tensor_at


def _torch():
    import torch
    return torch


class _Window(ctypes.Structure):
    _fields_ = [("peerPtr", ctypes.c_void_p * 8), ("mcPtr", ctypes.c_void_p), ("size", ctypes.c_size_t), ("rank", ctypes.c_int),
                ("nRanks", ctypes.c_int), ("userPtr", ctypes.c_void_p), ("devSelf", ctypes.c_void_p), ("hostState", ctypes.c_void_p),
                ("magic", ctypes.c_ulonglong)]


class _DevComm(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("nRanks", ctypes.c_int), ("lsaRank", ctypes.c_int), ("lsaSize", ctypes.c_int), ("resource", _Window),
                ("lsaBarrierOffset", ctypes.c_uint32), ("lsaBarrierCount", ctypes.c_int), ("llA2AOffset", ctypes.c_uint32),
                ("llA2ABlockCount", ctypes.c_int), ("llA2ASlotCount", ctypes.c_int), ("barrierEpochs", ctypes.c_void_p),
                ("llA2AEpochs", ctypes.c_void_p), ("ginSignalOffset", ctypes.c_uint32), ("ginSignalCount", ctypes.c_int),
                ("ginCounterOffset", ctypes.c_uint32), ("ginCounterCount", ctypes.c_int), ("abortFlag", ctypes.c_void_p),
                ("timeoutCycles", ctypes.c_ulonglong), ("ginProxyRing", ctypes.c_void_p), ("ginProxyHead", ctypes.c_void_p),
                ("ginProxyTail", ctypes.c_void_p), ("ginProxyDone", ctypes.c_void_p), ("ginProxyMask", ctypes.c_uint)]


class _Requirements(ctypes.Structure):
    _fields_ = [("size", ctypes.c_size_t), ("magic", ctypes.c_uint), ("version", ctypes.c_uint), ("resourceRequirementsList", ctypes.c_void_p),
                ("teamRequirementsList", ctypes.c_void_p)] + [(n, ctypes.c_int) for n in (
                    "lsaMultimem", "barrierCount", "lsaBarrierCount", "railGinBarrierCount", "lsaLLA2ABlockCount", "lsaLLA2ASlotCount",
                    "ginForceEnable", "ginContextCount", "ginSignalCount", "ginCounterCount", "ginConnectionType", "ginExclusiveContexts",
                    "ginQueueDepth", "ginTrafficClass", "worldGinBarrierCount", "ginStrongSignalsRequired", "ginVaSignalsRequired")]


class _Properties(ctypes.Structure):
    _fields_ = [("size", ctypes.c_size_t), ("magic", ctypes.c_uint), ("version", ctypes.c_uint)] + [(n, ctypes.c_int) for n in (
        "rank", "nRanks", "cudaDev", "nvmlDev", "deviceApiSupport", "multimemSupport", "ginType", "nLsaTeams", "hostRmaSupport", "railedGinType")]


def query_properties(comm):
    p = _Properties()
    p.size = ctypes.sizeof(_Properties)
    comm.lib.ncclCommQueryProperties.argtypes = [ctypes.c_void_p, ctypes.POINTER(_Properties)]
    _lib.check(comm.lib.ncclCommQueryProperties(comm.handle, ctypes.byref(p)), "ncclCommQueryProperties", comm.lib)
    return {n: getattr(p, n) for n, _ in _Properties._fields_[3:]}


class DeviceComm:
    def __init__(self, comm, barriers=64, ll_blocks=0, ll_slots=0, multimem=False, gin_signals=0, gin_counters=0):
        self.comm = comm
        self.lib = L = comm.lib
        L.ncclDevCommCreate.argtypes = [ctypes.c_void_p, ctypes.POINTER(_Requirements), ctypes.POINTER(_DevComm)]
        L.ncclDevCommDestroy.argtypes = [ctypes.c_void_p, ctypes.POINTER(_DevComm)]
        W, S, P = ctypes.POINTER(_Window), ctypes.c_size_t, ctypes.c_void_p
        L.b200DevApiAllReduce.argtypes = [ctypes.POINTER(_DevComm), W, S, W, S, S, ctypes.c_int, ctypes.c_int, ctypes.c_int, P]
        L.b200DevApiArRmsNorm.argtypes = [ctypes.POINTER(_DevComm), W, S, W, S, W, S, P, ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, P]
        L.b200DevApiLLSum.argtypes = [ctypes.POINTER(_DevComm), P, P, ctypes.c_int, ctypes.c_int, P]
        L.b200DevApiStatus.restype = ctypes.c_int
        L.b200DevApiGinRing.argtypes = [ctypes.POINTER(_DevComm), W, S, S, S, ctypes.c_ulonglong, P]
        req = _Requirements()
        req.size = ctypes.sizeof(_Requirements)
        req.magic = 0xdec0de01
        req.version = 23007
        req.lsaMultimem = int(multimem)
        req.lsaBarrierCount = barriers
        req.lsaLLA2ABlockCount = ll_blocks
        req.lsaLLA2ASlotCount = ll_slots
        req.ginContextCount = 4
        req.ginSignalCount = gin_signals
        req.ginCounterCount = gin_counters
        self._gin_seq = 0
        self.dc = _DevComm()
        _lib.check(L.ncclDevCommCreate(comm.handle, ctypes.byref(req), ctypes.byref(self.dc)), "ncclDevCommCreate", L)
        self.barriers = barriers
        self._wins = []      # (start, end, window pointer, raw allocation)

    def destroy(self):
        if self.dc is not None:
            _torch().cuda.synchronize()
            for _, _, win, ptr in self._wins:
                self.comm.deregister_window(win)
                mem_free(ptr, self.lib)
            self._wins = []
            _lib.check(self.lib.ncclDevCommDestroy(self.comm.handle, ctypes.byref(self.dc)), "ncclDevCommDestroy", self.lib)
            self.dc = None

    def symmetric(self, numel, dtype):
        """Tensor of `numel` elements over memory that every rank of the communicator can address."""
        torch = _torch()
        es = torch.empty(0, dtype=dtype).element_size()
        nbytes = max((numel * es + 255) // 256 * 256, 256)
        ptr = mem_alloc(nbytes, self.lib)
        raw = tensor_at(ptr, nbytes)
        win = self.comm.register_window(raw)
        self._wins.append((ptr, ptr + nbytes, win, ptr))
        return raw[:numel * es].view(dtype)

    def _locate(self, t):
        a = t.data_ptr()
        for lo, hi, win, _ in self._wins:
            if lo <= a and a + t.numel() * t.element_size() <= hi:
                return ctypes.cast(win, ctypes.POINTER(_Window)), a - lo
        raise ValueError("tensor does not live in a symmetric buffer of this device communicator")

    def _stream(self, stream):
        return (stream or _torch().cuda.current_stream()).cuda_stream

    def all_reduce(self, send, recv, multimem=False, ctas=32, stream=None):
        torch = _torch()
        code = {torch.float32: 7, torch.bfloat16: 9}[send.dtype]
        sw, so = self._locate(send)
        rw, ro = self._locate(recv)
        _lib.check(self.lib.b200DevApiAllReduce(ctypes.byref(self.dc), sw, so, rw, ro, send.numel(), code, int(multimem), min(ctas, self.barriers),
                                                self._stream(stream)), "b200DevApiAllReduce", self.lib)

    def ar_rmsnorm(self, partial, residual, out, weight, eps=1e-6, mode=0, ctas=64, stream=None):
        """out = rmsnorm(sum over ranks of partial + residual) * weight; residual is updated in place.
        mode 0: every rank reduces every row with peer loads; 1: the same through multimem; 2: rows
        dealt to ranks, owners store residual and out to every rank."""
        tokens, hidden = partial.shape
        iw, io = self._locate(partial)
        rw, ro = self._locate(residual)
        ow, oo = self._locate(out)
        _lib.check(self.lib.b200DevApiArRmsNorm(ctypes.byref(self.dc), iw, io, rw, ro, ow, oo, weight.data_ptr(), eps, tokens, hidden, mode,
                                                min(ctas, self.barriers), self._stream(stream)), "b200DevApiArRmsNorm", self.lib)

    def ll_sum(self, values, out, ctas=1, stream=None):
        """values, out: float32 [ctas, slots, 2]; out = sum over ranks (flagged-line all-to-all)."""
        slots = values.shape[1]
        _lib.check(self.lib.b200DevApiLLSum(ctypes.byref(self.dc), values.data_ptr(), out.data_ptr(), slots, ctas, self._stream(stream)),
                   "b200DevApiLLSum", self.lib)

    def gin_ring(self, send, recv, stream=None):
        """Every rank puts `send` into the next rank's `recv` (same symmetric buffer) and waits for its own to arrive."""
        sw, so = self._locate(send)
        rw, ro = self._locate(recv)
        if ctypes.addressof(sw.contents) != ctypes.addressof(rw.contents):
            raise ValueError("send and recv must live in the same symmetric buffer")
        self._gin_seq += 1
        _lib.check(self.lib.b200DevApiGinRing(ctypes.byref(self.dc), sw, so, ro, send.numel() * send.element_size(), self._gin_seq,
                                              self._stream(stream)), "b200DevApiGinRing", self.lib)

    def status(self):
        return self.lib.b200DevApiStatus()
