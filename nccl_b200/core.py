"""Communicators and collectives on torch tensors (GPU) or numpy arrays (host-memory communicators).

Thin object layer over the C API (reference shape: bindings/nccl4py/nccl/core/communicator.py):
one ``Communicator`` per rank, collectives take tensors, run on the current torch stream and
return immediately (stream-ordered).
"""
import contextlib
import ctypes

import numpy as np

from . import _lib

# ncclDataType_t
INT8, UINT8, INT32, UINT32, INT64, UINT64, FP16, FP32, FP64, BF16, FP8_E4M3, FP8_E5M2 = range(12)
# ncclRedOp_t
SUM, PROD, MAX, MIN, AVG = range(5)

_NP_TYPES = {np.dtype("int8"): INT8, np.dtype("uint8"): UINT8, np.dtype("int32"): INT32, np.dtype("uint32"): UINT32,
             np.dtype("int64"): INT64, np.dtype("uint64"): UINT64, np.dtype("float16"): FP16,
             np.dtype("float32"): FP32, np.dtype("float64"): FP64}
TYPE_SIZE = {INT8: 1, UINT8: 1, INT32: 4, UINT32: 4, INT64: 8, UINT64: 8, FP16: 2, FP32: 4, FP64: 8, BF16: 2, FP8_E4M3: 1, FP8_E5M2: 1}
_OPS = {"sum": SUM, "prod": PROD, "max": MAX, "min": MIN, "avg": AVG}


def _torch():
    import torch
    return torch


def _torch_types():
    torch = _torch()
    m = {torch.int8: INT8, torch.uint8: UINT8, torch.int32: INT32, torch.int64: INT64, torch.float16: FP16,
         torch.float32: FP32, torch.float64: FP64, torch.bfloat16: BF16}
    for name, code in (("float8_e4m3fn", FP8_E4M3), ("float8_e5m2", FP8_E5M2), ("uint32", UINT32), ("uint64", UINT64)):
        if hasattr(torch, name):
            m[getattr(torch, name)] = code
    return m


def describe(buf):
    """(pointer, element count, ncclDataType_t, is_cuda) of a tensor / array; None -> null pointer."""
    if buf is None:
        return 0, 0, None, False
    if isinstance(buf, np.ndarray):
        if not buf.flags["C_CONTIGUOUS"]:
            raise ValueError("numpy buffers must be C-contiguous")
        return buf.ctypes.data, buf.size, _NP_TYPES[buf.dtype], False
    if hasattr(buf, "data_ptr"):
        if not buf.is_contiguous():
            raise ValueError("tensors must be contiguous")
        return buf.data_ptr(), buf.numel(), _torch_types()[buf.dtype], buf.is_cuda
    raise TypeError("unsupported buffer type %r" % type(buf))


def _stream_of(buf, stream):
    if stream is not None:
        return stream if isinstance(stream, int) else stream.cuda_stream
    if buf is not None and hasattr(buf, "is_cuda") and buf.is_cuda:
        return _torch().cuda.current_stream(buf.device).cuda_stream
    return 0


def get_unique_id(lib=None):
    lib = lib or _lib.load()
    uid = _lib.ncclUniqueId()
    _lib.check(lib.ncclGetUniqueId(ctypes.byref(uid)), "ncclGetUniqueId", lib)
    return ctypes.string_at(ctypes.byref(uid), 128)   # (a c_char array read as .value would stop at the first NUL)


def unique_id_from_bytes(raw):
    uid = _lib.ncclUniqueId()
    ctypes.memmove(ctypes.byref(uid), raw, 128)
    return uid


def version(lib=None):
    v = ctypes.c_int()
    (lib or _lib.load()).ncclGetVersion(ctypes.byref(v))
    return v.value


@contextlib.contextmanager
def group(lib=None):
    """``with group(): ...`` brackets calls with ncclGroupStart / ncclGroupEnd."""
    lib = lib or _lib.load()
    _lib.check(lib.ncclGroupStart(), "ncclGroupStart", lib)
    try:
        yield
    finally:
        _lib.check(lib.ncclGroupEnd(), "ncclGroupEnd", lib)


class Communicator:
    """One rank of a communicator. ``lib`` selects the native library (default: this package's)."""

    def __init__(self, nranks, rank, unique_id, config=None, lib=None, _handle=None):
        self.lib = lib or _lib.load()
        self.nranks = nranks
        self.rank = rank
        self._windows = {}
        if _handle is not None:
            self.handle = _handle
            return
        h = _lib.ncclComm_t()
        uid = unique_id_from_bytes(unique_id) if isinstance(unique_id, (bytes, bytearray)) else unique_id
        if config is None:
            rc = self.lib.ncclCommInitRank(ctypes.byref(h), nranks, uid, rank)
        else:
            rc = self.lib.ncclCommInitRankConfig(ctypes.byref(h), nranks, uid, rank, ctypes.byref(config))
        _lib.check(rc, "ncclCommInitRank", self.lib)
        self.handle = h

    # ------------------------------------------------------------------ lifecycle
    def destroy(self):
        if self.handle:
            _lib.check(self.lib.ncclCommDestroy(self.handle), "ncclCommDestroy", self.lib)
            self.handle = None

    def abort(self):
        if self.handle:
            _lib.check(self.lib.ncclCommAbort(self.handle), "ncclCommAbort", self.lib)
            self.handle = None

    def finalize(self):
        _lib.check(self.lib.ncclCommFinalize(self.handle), "ncclCommFinalize", self.lib)

    def async_error(self):
        e = ctypes.c_int()
        _lib.check(self.lib.ncclCommGetAsyncError(self.handle, ctypes.byref(e)), "ncclCommGetAsyncError", self.lib)
        return e.value

    def split(self, color, key=0, config=None):
        h = _lib.ncclComm_t()
        rc = self.lib.ncclCommSplit(self.handle, color, key, ctypes.byref(h), ctypes.byref(config) if config else None)
        _lib.check(rc, "ncclCommSplit", self.lib)
        if not h.value:
            return None
        n, r = ctypes.c_int(), ctypes.c_int()
        self.lib.ncclCommCount(h, ctypes.byref(n))
        self.lib.ncclCommUserRank(h, ctypes.byref(r))
        return Communicator(n.value, r.value, None, lib=self.lib, _handle=h)

    def shrink(self, exclude, abort=False):
        arr = (ctypes.c_int * len(exclude))(*exclude)
        h = _lib.ncclComm_t()
        rc = self.lib.ncclCommShrink(self.handle, arr, len(exclude), ctypes.byref(h), None, 1 if abort else 0)
        _lib.check(rc, "ncclCommShrink", self.lib)
        n, r = ctypes.c_int(), ctypes.c_int()
        self.lib.ncclCommCount(h, ctypes.byref(n))
        self.lib.ncclCommUserRank(h, ctypes.byref(r))
        return Communicator(n.value, r.value, None, lib=self.lib, _handle=h)

    # ------------------------------------------------------------------ memory
    def register_window(self, tensor, symmetric=True):
        """Collective: makes ``tensor``'s memory addressable by every rank (zero-copy collectives)."""
        ptr, n, dt, _ = describe(tensor)
        win = ctypes.c_void_p()
        rc = self.lib.ncclCommWindowRegister(self.handle, ptr, n * TYPE_SIZE[dt], ctypes.byref(win), 1 if symmetric else 0)
        _lib.check(rc, "ncclCommWindowRegister", self.lib)
        self._windows[ptr] = win
        return win

    def deregister_window(self, win):
        _lib.check(self.lib.ncclCommWindowDeregister(self.handle, win), "ncclCommWindowDeregister", self.lib)
        for k, v in list(self._windows.items()):
            if v.value == win.value:
                del self._windows[k]

    def mem_stats(self, stat):
        v = ctypes.c_uint64()
        _lib.check(self.lib.ncclCommMemStats(self.handle, stat, ctypes.byref(v)), "ncclCommMemStats", self.lib)
        return v.value

    def suspend(self):
        _lib.check(self.lib.ncclCommSuspend(self.handle, 1), "ncclCommSuspend", self.lib)

    def resume(self):
        _lib.check(self.lib.ncclCommResume(self.handle), "ncclCommResume", self.lib)

    # ------------------------------------------------------------------ reduction operators
    def _op(self, op):
        return _OPS[op] if isinstance(op, str) else int(op)

    def premul_sum(self, scalar, dtype_code):
        """Creates a pre-multiplied-sum operator from a host scalar; returns the operator handle."""
        np_type = {FP32: np.float32, FP64: np.float64, FP16: np.float16, INT32: np.int32, INT64: np.int64}.get(dtype_code)
        if np_type is not None:
            raw = np.array([scalar], dtype=np_type).tobytes()
        elif dtype_code == BF16:
            raw = (np.array([scalar], dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes()
        else:
            raise ValueError("premul_sum: unsupported type")
        buf = ctypes.create_string_buffer(raw, 8)
        op = ctypes.c_int()
        _lib.check(self.lib.ncclRedOpCreatePreMulSum(ctypes.byref(op), buf, dtype_code, 1, self.handle), "ncclRedOpCreatePreMulSum", self.lib)
        return op.value

    def destroy_op(self, op):
        _lib.check(self.lib.ncclRedOpDestroy(op, self.handle), "ncclRedOpDestroy", self.lib)

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, send, recv=None, op="sum", stream=None):
        recv = send if recv is None else recv
        sp, n, dt, _ = describe(send)
        rp = describe(recv)[0]
        _lib.check(self.lib.ncclAllReduce(sp, rp, n, dt, self._op(op), self.handle, _stream_of(send, stream)), "ncclAllReduce", self.lib)
        return recv

    def all_reduce_from_host(self, host_send, host_recv, dev_send, dev_recv=None, op="sum", stream=None, chunk_bytes=0):
        """All-reduce of pinned host tensors through device staging buffers, chunked so that the copy in, the
        collective and the copy out of neighbouring chunks overlap (ncclAllReduceFromHost). Work queued on the
        stream afterwards, and an event recorded on it, comes after the last byte has reached ``host_recv``."""
        dev_recv = dev_send if dev_recv is None else dev_recv
        if not (host_send.is_pinned() and host_recv.is_pinned()):
            raise ValueError("host tensors must be pinned")
        _, n, dt, _ = describe(dev_send)
        if host_send.numel() * host_send.element_size() != dev_send.numel() * dev_send.element_size():
            raise ValueError("host and device buffers differ in size")
        fn = self.lib.ncclAllReduceFromHost
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
        _lib.check(fn(host_send.data_ptr(), host_recv.data_ptr(), dev_send.data_ptr(), dev_recv.data_ptr(), n, dt, self._op(op), self.handle,
                      _stream_of(dev_send, stream), chunk_bytes), "ncclAllReduceFromHost", self.lib)
        return host_recv

    def reduce(self, send, recv, root, op="sum", stream=None):
        sp, n, dt, _ = describe(send)
        rp = describe(recv)[0]
        _lib.check(self.lib.ncclReduce(sp, rp, n, dt, self._op(op), root, self.handle, _stream_of(send, stream)), "ncclReduce", self.lib)
        return recv

    def broadcast(self, send, recv, root, stream=None):
        ref = recv if recv is not None else send
        sp = describe(send)[0]
        rp, n, dt, _ = describe(ref)
        _lib.check(self.lib.ncclBroadcast(sp, rp, n, dt, root, self.handle, _stream_of(ref, stream)), "ncclBroadcast", self.lib)
        return recv

    def reduce_scatter(self, send, recv, op="sum", stream=None):
        sp = describe(send)[0]
        rp, n, dt, _ = describe(recv)
        _lib.check(self.lib.ncclReduceScatter(sp, rp, n, dt, self._op(op), self.handle, _stream_of(send, stream)), "ncclReduceScatter", self.lib)
        return recv

    def all_gather(self, send, recv, stream=None):
        sp, n, dt, _ = describe(send)
        rp = describe(recv)[0]
        _lib.check(self.lib.ncclAllGather(sp, rp, n, dt, self.handle, _stream_of(send, stream)), "ncclAllGather", self.lib)
        return recv

    def all_to_all(self, send, recv, stream=None):
        sp, n, dt, _ = describe(send)
        rp = describe(recv)[0]
        _lib.check(self.lib.ncclAlltoAll(sp, rp, n // self.nranks, dt, self.handle, _stream_of(send, stream)), "ncclAlltoAll", self.lib)
        return recv

    def gather(self, send, recv, root, stream=None):
        sp, n, dt, _ = describe(send)
        rp = describe(recv)[0]
        _lib.check(self.lib.ncclGather(sp, rp, n, dt, root, self.handle, _stream_of(send, stream)), "ncclGather", self.lib)
        return recv

    def scatter(self, send, recv, root, stream=None):
        sp = describe(send)[0]
        rp, n, dt, _ = describe(recv)
        _lib.check(self.lib.ncclScatter(sp, rp, n, dt, root, self.handle, _stream_of(recv, stream)), "ncclScatter", self.lib)
        return recv

    def send(self, buf, peer, stream=None):
        p, n, dt, _ = describe(buf)
        _lib.check(self.lib.ncclSend(p, n, dt, peer, self.handle, _stream_of(buf, stream)), "ncclSend", self.lib)

    def recv(self, buf, peer, stream=None):
        p, n, dt, _ = describe(buf)
        _lib.check(self.lib.ncclRecv(p, n, dt, peer, self.handle, _stream_of(buf, stream)), "ncclRecv", self.lib)
        return buf


def mem_alloc(nbytes, lib=None):
    lib = lib or _lib.load()
    p = ctypes.c_void_p()
    _lib.check(lib.ncclMemAlloc(ctypes.byref(p), nbytes), "ncclMemAlloc", lib)
    return p.value


def mem_free(ptr, lib=None):
    lib = lib or _lib.load()
    _lib.check(lib.ncclMemFree(ctypes.c_void_p(ptr)), "ncclMemFree", lib)
