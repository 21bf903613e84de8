"""``nccl.core`` of the reference's Python bindings, re-stated over :mod:`nccl_b200.core`.

Same class and method names, keyword arguments and return conventions (collectives return ``None``; buffers are
anything that exposes ``data_ptr`` / ``__cuda_array_interface__`` through :func:`nccl_b200.core.describe`, i.e. torch
tensors and numpy arrays here; streams are ``None``, an integer handle or an object with ``cuda_stream``).
Reference parity: bindings/nccl4py/nccl/core/communicator.py (Communicator: init / init_all / split / shrink / grow /
destroy / abort / finalize / revoke / suspend / resume, properties, send / recv / allreduce / broadcast / reduce /
allgather / reduce_scatter / alltoall / gather / scatter, register_buffer / register_window, create_pre_mul_sum,
get_async_error, get_mem_stat), group.py (group), memory.py (mem_alloc / mem_free), utils.py (get_unique_id, get_version).
"""
import contextlib
import ctypes
import enum

from ... import _lib
from ... import core as _core

__all__ = ["Communicator", "NCCLConfig", "UniqueId", "NcclRedOp", "SUM", "PROD", "MAX", "MIN", "AVG", "NcclCommMemStat", "CommSuspendFlag",
           "WindowFlag", "get_unique_id", "get_version", "group", "group_start", "group_end", "mem_alloc", "mem_free", "NcclError"]


class NcclError(RuntimeError):
    """Raised when a library call returns anything but success."""


class NcclRedOp(enum.IntEnum):
    SUM = 0
    PROD = 1
    MAX = 2
    MIN = 3
    AVG = 4


SUM, PROD, MAX, MIN, AVG = NcclRedOp.SUM, NcclRedOp.PROD, NcclRedOp.MAX, NcclRedOp.MIN, NcclRedOp.AVG


class NcclCommMemStat(enum.IntEnum):
    GPU_MEM_SUSPEND = 0
    GPU_MEM_SUSPENDED = 1
    GPU_MEM_PERSIST = 2
    GPU_MEM_TOTAL = 3


class CommSuspendFlag(enum.IntFlag):
    MEM = 1


class WindowFlag(enum.IntFlag):
    DEFAULT = 0
    COLL_SYMMETRIC = 1


class UniqueId:
    """128 opaque bytes that every rank passes to :meth:`Communicator.init`."""

    def __init__(self, raw=None):
        self.raw = bytes(raw) if raw is not None else bytes(128)

    def __bytes__(self):
        return self.raw

    @classmethod
    def from_bytes(cls, raw):
        return cls(raw)

    def as_bytes(self):
        return self.raw


class NCCLConfig:
    """Keyword view of ncclConfig_t: unset fields keep the library's defaults."""
    FIELDS = ("blocking", "cga_cluster_size", "min_ctas", "max_ctas", "net_name", "split_share", "traffic_class", "comm_name")

    def __init__(self, **kw):
        for k in kw:
            if k not in self.FIELDS:
                raise TypeError("unknown configuration field %r" % k)
        self.values = dict(kw)

    def to_struct(self):
        cfg = _core.Config() if hasattr(_core, "Config") else None
        if cfg is None:
            return None
        names = {"blocking": "blocking", "cga_cluster_size": "cgaClusterSize", "min_ctas": "minCTAs", "max_ctas": "maxCTAs",
                 "split_share": "splitShare", "traffic_class": "trafficClass"}
        for k, v in self.values.items():
            if k in names and hasattr(cfg, names[k]):
                setattr(cfg, names[k], int(v))
        return cfg


def get_unique_id():
    return UniqueId(_core.get_unique_id())


def get_version():
    v = ctypes.c_int()
    lib = _lib.load()
    _lib.check(lib.ncclGetVersion(ctypes.byref(v)), "ncclGetVersion", lib)
    return v.value


def group_start():
    lib = _lib.load()
    _lib.check(lib.ncclGroupStart(), "ncclGroupStart", lib)


def group_end():
    lib = _lib.load()
    _lib.check(lib.ncclGroupEnd(), "ncclGroupEnd", lib)


@contextlib.contextmanager
def group():
    group_start()
    try:
        yield
    finally:
        group_end()


def mem_alloc(nbytes):
    """Device memory that windows can be registered over (ncclMemAlloc); returns the address."""
    return _core.mem_alloc(nbytes)


def mem_free(ptr):
    _core.mem_free(ptr)


class RegisteredBufferHandle:
    def __init__(self, comm, handle):
        self._comm, self.handle = comm, handle

    def close(self):
        if self.handle is not None:
            lib = self._comm._c.lib
            _lib.check(lib.ncclCommDeregister(self._comm._c.handle, self.handle), "ncclCommDeregister", lib)
            self.handle = None


class RegisteredWindowHandle:
    def __init__(self, comm, win):
        self._comm, self.handle = comm, win

    def close(self):
        if self.handle is not None:
            self._comm._c.deregister_window(self.handle)
            self.handle = None


class CustomRedOp:
    """A pre-multiplied sum created by :meth:`Communicator.create_pre_mul_sum`."""

    def __init__(self, comm, op):
        self._comm, self.op = comm, op

    def close(self):
        if self.op is not None:
            self._comm._c.destroy_op(self.op)
            self.op = None

    def __int__(self):
        return int(self.op)


class Communicator:
    """One rank of a communicator, with the reference bindings' method names."""

    def __init__(self, ptr=0):
        self._c = None
        self._resources = []

    # ------------------------------------------------------------------ creation
    @classmethod
    def init(cls, nranks, rank, unique_id, config=None):
        comm = cls()
        comm.initialize(nranks, rank, unique_id, config)
        return comm

    def initialize(self, nranks, rank, unique_id, config=None):
        if isinstance(unique_id, (list, tuple)):
            unique_id = unique_id[0]   # several roots only spread the rendezvous load; one root serves any size here
        raw = bytes(unique_id) if not isinstance(unique_id, (bytes, bytearray)) else unique_id
        cfg = config.to_struct() if isinstance(config, NCCLConfig) else config
        self._c = _core.Communicator(nranks, rank, raw, config=cfg)

    @classmethod
    def _wrap(cls, inner):
        if inner is None:
            return None
        comm = cls()
        comm._c = inner
        return comm

    def split(self, color, key=0, config=None):
        return self._wrap(self._c.split(-1 if color is None else color, key))

    @classmethod
    def init_all(cls, devices=None):
        """One communicator per listed device of this process (all visible devices by default): ncclCommInitAll."""
        lib = _lib.load()
        if devices is None:
            import torch
            devices = list(range(torch.cuda.device_count()))
        n = len(devices)
        handles = (ctypes.c_void_p * n)()
        lib.ncclCommInitAll.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        _lib.check(lib.ncclCommInitAll(handles, n, (ctypes.c_int * n)(*devices)), "ncclCommInitAll", lib)
        return [cls._wrap(_core.Communicator(n, r, None, lib=lib, _handle=ctypes.c_void_p(handles[r]))) for r in range(n)]

    def grow(self, nranks, unique_id=None, rank=-1, config=None):
        """ncclCommGrow: the ranks of this communicator (which pass rank = -1 and, except the one that made it, no id)
        and new ranks (which pass their rank and the id, on a communicator object without a parent) form a larger one."""
        lib = _lib.load() if self._c is None else self._c.lib
        new = ctypes.c_void_p()
        uid = None
        if unique_id is not None:
            uid = _lib.ncclUniqueId.from_buffer_copy(bytes(unique_id))
        lib.ncclCommGrow.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
        parent = self._c.handle if self._c is not None else None
        _lib.check(lib.ncclCommGrow(parent, nranks, ctypes.byref(uid) if uid is not None else None, rank, ctypes.byref(new), None), "ncclCommGrow", lib)
        r = ctypes.c_int()
        lib.ncclCommUserRank(new, ctypes.byref(r))
        return self._wrap(_core.Communicator(nranks, r.value, None, lib=lib, _handle=new))

    def shrink(self, exclude_ranks, config=None, flags=0):
        return self._wrap(self._c.shrink(list(exclude_ranks), abort=bool(flags)))

    def get_unique_id(self):
        uid = _lib.ncclUniqueId()
        lib = self._c.lib
        _lib.check(lib.ncclCommGetUniqueId(self._c.handle, ctypes.byref(uid)), "ncclCommGetUniqueId", lib)
        return UniqueId(ctypes.string_at(ctypes.byref(uid), 128))

    # ------------------------------------------------------------------ teardown and state
    def _check_valid(self, operation):
        if self._c is None or not self._c.handle:
            raise NcclError("%s on a communicator that was destroyed or never initialised" % operation)

    def close_all_resources(self):
        for r in self._resources:
            r.close()
        self._resources = []

    def destroy(self):
        if self._c is not None:
            self.close_all_resources()
            self._c.destroy()

    def abort(self):
        if self._c is not None:
            self._c.abort()

    def finalize(self):
        self._check_valid("finalize")
        self._c.finalize()

    def revoke(self, flags=0):
        self._check_valid("revoke")
        lib = self._c.lib
        _lib.check(lib.ncclCommRevoke(self._c.handle, int(flags)), "ncclCommRevoke", lib)

    def suspend(self, flags=CommSuspendFlag.MEM):
        self._check_valid("suspend")
        self._c.suspend()

    def resume(self):
        self._check_valid("resume")
        self._c.resume()

    @property
    def ptr(self):
        return self._c.handle.value if self._c is not None and self._c.handle else 0

    @property
    def is_valid(self):
        return self.ptr != 0

    @property
    def nranks(self):
        return self._c.nranks

    @property
    def rank(self):
        return self._c.rank

    @property
    def cuda_dev(self):
        d = ctypes.c_int()
        _lib.check(self._c.lib.ncclCommCuDevice(self._c.handle, ctypes.byref(d)), "ncclCommCuDevice", self._c.lib)
        return d.value

    @property
    def device(self):
        """CUDA device ordinal of this rank (the reference returns a device object; the ordinal identifies it)."""
        return self.cuda_dev

    def _properties(self):
        from ...ops.devapi import query_properties
        return query_properties(self._c)

    @property
    def nvml_dev(self):
        return self._properties()["nvmlDev"]

    @property
    def gin_type(self):
        return self._properties()["ginType"]

    @property
    def railed_gin_type(self):
        return self._properties()["railedGinType"]

    @property
    def n_lsa_teams(self):
        return self._properties()["nLsaTeams"]

    @property
    def host_rma_support(self):
        return bool(self._properties()["hostRmaSupport"])

    @property
    def multimem_support(self):
        fn = self._c.lib.b200CommHasMulticast
        fn.argtypes = [ctypes.c_void_p]
        return bool(fn(self._c.handle))

    @property
    def device_api_support(self):
        fn = self._c.lib.b200CommIsSymmetric
        fn.argtypes = [ctypes.c_void_p]
        return bool(fn(self._c.handle))

    def get_async_error(self):
        return self._c.async_error()

    def get_last_error(self):
        fn = self._c.lib.ncclGetLastError
        fn.restype = ctypes.c_char_p
        fn.argtypes = [ctypes.c_void_p]
        return (fn(self._c.handle) or b"").decode()

    def get_mem_stat(self, stat):
        return self._c.mem_stats(int(stat))

    # ------------------------------------------------------------------ point to point and one-sided
    def send(self, sendbuf, peer, *, stream=None):
        self._check_valid("send")
        self._c.send(sendbuf, peer, stream=stream)

    def recv(self, recvbuf, peer, *, stream=None):
        self._check_valid("recv")
        self._c.recv(recvbuf, peer, stream=stream)

    def put_signal(self, sendbuf, peer, peer_window, peer_offset=0, *, sig_idx=0, ctx=0, flags=0, stream=None):
        """One-sided: copies ``sendbuf`` into ``peer``'s part of a registered window and bumps its signal ``sig_idx``."""
        self._check_valid("put_signal")
        ptr, n, dt, _ = _core.describe(sendbuf)
        lib = self._c.lib
        lib.ncclPutSignal.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p]
        win = getattr(peer_window, "handle", peer_window)
        _lib.check(lib.ncclPutSignal(ptr, n, dt, peer, win, peer_offset, sig_idx, ctx, flags, self._c.handle, _core._stream_of(sendbuf, stream)),
                   "ncclPutSignal", lib)

    def signal(self, peer, *, sig_idx=0, ctx=0, flags=0, stream=None):
        self._check_valid("signal")
        lib = self._c.lib
        lib.ncclSignal.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p]
        _lib.check(lib.ncclSignal(peer, sig_idx, ctx, flags, self._c.handle, _core._stream_of(None, stream)), "ncclSignal", lib)

    def wait_signal(self, descs, *, stream=None):
        """``descs``: iterable of (peer, op_count[, sig_idx[, ctx]]): waits until each peer has signalled that many times more."""
        self._check_valid("wait_signal")

        class _Desc(ctypes.Structure):
            _fields_ = [("opCnt", ctypes.c_int), ("peer", ctypes.c_int), ("sigIdx", ctypes.c_int), ("ctx", ctypes.c_int)]

        items = []
        for d in descs:
            d = tuple(d) + (0, 0)
            items.append(_Desc(int(d[1]), int(d[0]), int(d[2]), int(d[3])))
        arr = (_Desc * len(items))(*items)
        lib = self._c.lib
        lib.ncclWaitSignal.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        _lib.check(lib.ncclWaitSignal(len(items), arr, self._c.handle, _core._stream_of(None, stream)), "ncclWaitSignal", lib)

    def create_dev_comm(self, **requirements):
        """A device communicator for kernels written with the device API (``nccl_b200.ops.devapi.DeviceComm`` keywords:
        barriers, ll_blocks, ll_slots, gin_signals, gin_counters, multimem)."""
        from ...ops.devapi import DeviceComm
        dc = DeviceComm(self._c, **requirements)
        self._resources.append(type("DevCommResource", (), {"close": lambda s, d=dc: d.destroy()})())
        return dc

    # ------------------------------------------------------------------ collectives
    def reduce(self, sendbuf, recvbuf, op, *, root=None, stream=None):
        """``root=None`` reduces to every rank (all-reduce), as in the reference bindings."""
        self._check_valid("reduce")
        if root is None:
            self._c.all_reduce(sendbuf, recvbuf, op=int(op), stream=stream)
        else:
            self._c.reduce(sendbuf, recvbuf, root, op=int(op), stream=stream)

    def allreduce(self, sendbuf, recvbuf, op, *, stream=None):
        self.reduce(sendbuf, recvbuf, op, stream=stream)

    def broadcast(self, sendbuf, recvbuf, root, *, stream=None):
        self._check_valid("broadcast")
        self._c.broadcast(sendbuf if sendbuf is not None else recvbuf, recvbuf, root, stream=stream)

    def allgather(self, sendbuf, recvbuf, *, stream=None):
        self._check_valid("allgather")
        self._c.all_gather(sendbuf, recvbuf, stream=stream)

    def reduce_scatter(self, sendbuf, recvbuf, op, *, stream=None):
        self._check_valid("reduce_scatter")
        self._c.reduce_scatter(sendbuf, recvbuf, op=int(op), stream=stream)

    def alltoall(self, sendbuf, recvbuf, *, stream=None):
        self._check_valid("alltoall")
        self._c.all_to_all(sendbuf, recvbuf, stream=stream)

    def gather(self, sendbuf, recvbuf, root, *, stream=None):
        self._check_valid("gather")
        self._c.gather(sendbuf, recvbuf if recvbuf is not None else sendbuf, root, stream=stream)

    def scatter(self, sendbuf, recvbuf, root, *, stream=None):
        self._check_valid("scatter")
        self._c.scatter(sendbuf if sendbuf is not None else recvbuf, recvbuf, root, stream=stream)

    # ------------------------------------------------------------------ registration and operators
    def register_buffer(self, buffer):
        self._check_valid("register_buffer")
        ptr, n, dt, _ = _core.describe(buffer)
        h = ctypes.c_void_p()
        lib = self._c.lib
        _lib.check(lib.ncclCommRegister(self._c.handle, ctypes.c_void_p(ptr), n * _core.TYPE_SIZE[dt], ctypes.byref(h)), "ncclCommRegister", lib)
        res = RegisteredBufferHandle(self, h)
        self._resources.append(res)
        return res

    def register_window(self, buffer, flags=WindowFlag.COLL_SYMMETRIC):
        self._check_valid("register_window")
        res = RegisteredWindowHandle(self, self._c.register_window(buffer, symmetric=bool(int(flags) & 1)))
        self._resources.append(res)
        return res

    def create_pre_mul_sum(self, scalar, datatype):
        self._check_valid("create_pre_mul_sum")
        res = CustomRedOp(self, self._c.premul_sum(scalar, int(datatype)))
        self._resources.append(res)
        return res

    def __repr__(self):
        return "<Communicator rank %s of %s, %s>" % (getattr(self._c, "rank", "?"), getattr(self._c, "nranks", "?"), "valid" if self.is_valid else "closed")
