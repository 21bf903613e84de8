"""Expert-parallel dispatch / combine with the call shapes of the reference's ``nccl.ep`` Python package
(``Group.create``, ``group.create_handle``, ``handle.dispatch / combine / complete``, ``Tensor`` descriptors and the
configuration records) over this library's ncclEp* entry points.

    group = ep.Group.create(comm, ep.GroupConfig(num_experts=256, max_dispatch_tokens_per_rank=4096, max_token_bytes=2 * 7168))
    handle = group.create_handle(ep.Layout.EXPERT_MAJOR, ep.Tensor(topk_idx), stream=stream)
    handle.dispatch(ep.DispatchInputs(tokens=ep.Tensor(x), topk_weights=ep.Tensor(w)),
                    ep.DispatchOutputs(tokens=ep.Tensor(toks), scales=ep.Tensor(scales)),
                    layout_info=ep.LayoutInfo(expert_counters=ep.Tensor(counts)), stream=stream)
    handle.combine(ep.CombineInputs(tokens=ep.Tensor(y)), ep.CombineOutputs(tokens=ep.Tensor(out)), stream=stream)

Reference parity: bindings/nccl4py/nccl/ep/{group,handle,tensor,enums}.py.
"""
import ctypes
from dataclasses import dataclass, field
from enum import IntEnum

from .. import _lib
from ..core import describe
from ..ops import ep as _ep


class Algorithm(IntEnum):
    LOW_LATENCY = 0
    HIGH_THROUGHPUT = 1


class Layout(IntEnum):
    UNSET = 0
    EXPERT_MAJOR = 1
    RANK_MAJOR = 2
    FLAT = 3


class PassDir(IntEnum):
    FWD = 0
    BWD = 1


def _stream_ptr(stream):
    if stream is None:
        return None
    return stream if isinstance(stream, int) else getattr(stream, "cuda_stream", getattr(stream, "ptr", stream))


class Tensor:
    """Descriptor of a buffer for the ncclEp* calls: data pointer, shape and element type of anything ``describe`` understands
    (torch tensors, numpy arrays, objects with ``__cuda_array_interface__``)."""

    def __init__(self, buffer, datatype=None):
        self._buffer = buffer
        ptr, n, dt, _ = describe(buffer)
        self._shape = tuple(int(s) for s in buffer.shape)
        self._dt = dt if datatype is None else int(datatype)
        self._sizes = (ctypes.c_size_t * len(self._shape))(*self._shape)
        self._c = _ep.EpTensor(ctypes.sizeof(_ep.EpTensor), _ep.TENSOR_MAGIC, len(self._shape), self._dt, ptr, None, 0, self._sizes)

    @property
    def ptr(self):
        return ctypes.addressof(self._c)

    @property
    def ndim(self):
        return len(self._shape)

    @property
    def sizes(self):
        return self._shape

    @property
    def datatype(self):
        return self._dt

    @property
    def data(self):
        return self._c.data

    @property
    def buffer(self):
        return self._buffer

    def _pointer(self):
        return ctypes.pointer(self._c)

    def __repr__(self):
        return "Tensor(shape=%s, datatype=%d, data=0x%x)" % (self._shape, self._dt, self._c.data or 0)


def _p(t):
    return t._pointer() if t is not None else None


AllocFn = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t, ctypes.c_void_p)   # cudaError_t (*)(void** ptr, size_t size, void* context)
FreeFn = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p)                                      # cudaError_t (*)(void* ptr, void* context)


@dataclass
class AllocConfig:
    """Addresses of C-callable allocator hooks (``ctypes.cast(fn, ctypes.c_void_p).value`` of an ``AllocFn`` / ``FreeFn`` or of a
    symbol of a shared library) for the buffers that only this rank touches; 0 leaves them to cudaMalloc / cudaFree. Memory
    that peers map always comes from the library's own allocator. The callables must stay alive as long as the group."""
    alloc_fn: int = 0
    free_fn: int = 0
    context: int = 0


def get_lib_version():
    """Version of the expert-parallel API in the loaded library as ``(major, minor, patch)``."""
    lib = _lib.load()
    v = ctypes.c_int(0)
    _lib.check(lib.ncclEpGetVersion(ctypes.byref(v)), "ncclEpGetVersion", lib)
    return (v.value // 10000, (v.value % 10000) // 100, v.value % 100)


def get_lib_path():
    """Path of the loaded shared library (the expert-parallel entry points live in the main library)."""
    import pathlib
    return pathlib.Path(_lib.load()._name)


def get_nccl_comm_from_group(group=None):
    """A new communicator with the membership of a ``torch.distributed`` process group (the default group when ``None``): the
    group's first rank makes the unique id and broadcasts its bytes through the process group."""
    import torch
    import torch.distributed as dist
    from . import core as nccl
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised: call init_process_group first")
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    src = dist.get_process_group_ranks(group)[0] if group is not None else 0
    box = [nccl.get_unique_id().as_bytes() if rank == 0 else None]
    dist.broadcast_object_list(box, src=src, group=group)
    return nccl.Communicator.init(world, rank, nccl.UniqueId(box[0]))


@dataclass
class GroupConfig:
    algorithm: Algorithm = Algorithm.LOW_LATENCY
    num_experts: int = 0
    max_dispatch_tokens_per_rank: int = 0
    max_recv_tokens_per_rank: int = 0
    max_token_bytes: int = 0
    rdma_buffer_size: int = 0
    num_qp_per_rank: int = 0
    num_channels: int = 0
    max_num_sms: int = 0
    alloc: AllocConfig = field(default_factory=AllocConfig)
    enable_mask: bool = False
    timeout_ns: int = 0


@dataclass
class HandleConfig:
    dispatch_output_per_expert_alignment: int = 0


@dataclass
class DispatchConfig:
    send_only: int = 0
    round_scales: int = 0
    pass_direction: PassDir = PassDir.FWD


@dataclass
class CombineConfig:
    send_only: int = 0
    pass_direction: PassDir = PassDir.FWD


@dataclass
class LayoutInfo:
    expert_counters: Tensor = None
    src_rank_counters: Tensor = None
    expert_offsets: Tensor = None
    recv_total_counter: Tensor = None

    def _struct(self):
        li = _ep._hdr(_ep.LayoutInfo())
        li.expert_counters, li.src_rank_counters = _p(self.expert_counters), _p(self.src_rank_counters)
        li.expert_offsets, li.recv_total_counter = _p(self.expert_offsets), _p(self.recv_total_counter)
        return li


@dataclass
class DispatchInputs:
    tokens: Tensor = None
    topk_weights: Tensor = None
    scales: Tensor = None


@dataclass
class DispatchOutputs:
    tokens: Tensor = None
    topk_weights: Tensor = None
    scales: Tensor = None
    topk_idx: Tensor = None


@dataclass
class CombineInputs:
    tokens: Tensor = None
    topk_weights: Tensor = None


@dataclass
class CombineOutputs:
    tokens: Tensor = None
    topk_weights: Tensor = None


class _HandleCfg(ctypes.Structure):
    _fields_ = [("size", ctypes.c_uint), ("magic", ctypes.c_uint), ("dispatch_output_per_expert_alignment", ctypes.c_size_t)]


class Handle:
    def __init__(self, ptr, lib):
        self._ptr, self._lib = ptr, lib
        self._keep = None

    def _check_valid(self, operation):
        if not self._ptr:
            raise RuntimeError("%s on a handle that was destroyed" % operation)

    @property
    def ptr(self):
        return self._ptr.value if self._ptr else 0

    def update(self, topk_idx, *, layout_info=None, stream=None):
        self._check_valid("update")
        li = layout_info._struct() if layout_info is not None else None
        _lib.check(self._lib.ncclEpUpdateHandle(self._ptr, _p(topk_idx), ctypes.byref(li) if li is not None else None, _stream_ptr(stream)),
                   "ncclEpUpdateHandle", self._lib)
        self._keep = (topk_idx, layout_info, li)

    def dispatch(self, inputs, outputs, *, layout_info=None, config=None, stream=None):
        self._check_valid("dispatch")
        din, dout = _ep._hdr(_ep.DispIn()), _ep._hdr(_ep.DispOut())
        din.tokens, din.topk_weights, din.scales = _p(inputs.tokens), _p(inputs.topk_weights), _p(inputs.scales)
        dout.tokens, dout.topk_weights, dout.scales, dout.topk_idx = _p(outputs.tokens), _p(outputs.topk_weights), _p(outputs.scales), _p(outputs.topk_idx)
        li = layout_info._struct() if layout_info is not None else None
        cfg = _ep._hdr(_ep.DispCfg())
        if config is not None:
            cfg.send_only, cfg.round_scales, cfg.pass_direction = int(config.send_only), int(config.round_scales), int(config.pass_direction)
        _lib.check(self._lib.ncclEpDispatch(self._ptr, ctypes.byref(din), ctypes.byref(dout), ctypes.byref(li) if li is not None else None,
                                            ctypes.byref(cfg), _stream_ptr(stream)), "ncclEpDispatch", self._lib)
        self._keep_d = (inputs, outputs, layout_info, li)

    def combine(self, inputs, outputs, *, config=None, stream=None):
        self._check_valid("combine")
        cin, cout = _ep._hdr(_ep.CombIO()), _ep._hdr(_ep.CombIO())
        cin.tokens, cin.topk_weights = _p(inputs.tokens), _p(inputs.topk_weights)
        cout.tokens, cout.topk_weights = _p(outputs.tokens), _p(outputs.topk_weights)
        cfg = _ep._hdr(_ep.CombCfg())
        if config is not None:
            cfg.send_only, cfg.pass_direction = int(config.send_only), int(config.pass_direction)
        _lib.check(self._lib.ncclEpCombine(self._ptr, ctypes.byref(cin), ctypes.byref(cout), ctypes.byref(cfg), _stream_ptr(stream)), "ncclEpCombine", self._lib)
        self._keep_c = (inputs, outputs)

    def complete(self, *, config=0, stream=None):
        self._check_valid("complete")
        if config:
            raise ValueError("complete: config is reserved and must be 0")
        _lib.check(self._lib.ncclEpComplete(self._ptr, None, _stream_ptr(stream)), "ncclEpComplete", self._lib)

    def destroy(self):
        if self._ptr:
            self._lib.ncclEpHandleDestroy(self._ptr)
            self._ptr = None

    def __repr__(self):
        return "Handle(ptr=0x%x)" % self.ptr


class Group:
    def __init__(self, ptr, lib):
        self._ptr, self._lib = ptr, lib

    @classmethod
    def create(cls, comm, config):
        inner = getattr(comm, "_c", comm)   # a nccl4py Communicator or the package's own
        lib = inner.lib
        vp, pvp = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)
        lib.ncclEpCreateGroup.argtypes = [pvp, vp, ctypes.POINTER(_ep.GroupCfg)]
        lib.ncclEpGroupDestroy.argtypes = [vp]
        lib.ncclEpCreateHandle.argtypes = [pvp, vp, ctypes.c_int, ctypes.POINTER(_ep.EpTensor), vp, vp, vp]
        lib.ncclEpUpdateHandle.argtypes = [vp, ctypes.POINTER(_ep.EpTensor), vp, vp]
        lib.ncclEpHandleDestroy.argtypes = [vp]
        lib.ncclEpDispatch.argtypes = [vp, ctypes.POINTER(_ep.DispIn), ctypes.POINTER(_ep.DispOut), ctypes.POINTER(_ep.LayoutInfo), ctypes.POINTER(_ep.DispCfg), vp]
        lib.ncclEpCombine.argtypes = [vp, ctypes.POINTER(_ep.CombIO), ctypes.POINTER(_ep.CombIO), ctypes.POINTER(_ep.CombCfg), vp]
        lib.ncclEpComplete.argtypes = [vp, vp, vp]
        cfg = _ep._hdr(_ep.GroupCfg())
        cfg.version = 1
        cfg.algorithm = int(config.algorithm)
        for name in ("num_experts", "max_dispatch_tokens_per_rank", "max_recv_tokens_per_rank", "max_token_bytes", "rdma_buffer_size", "num_qp_per_rank",
                     "num_channels", "max_num_sms", "timeout_ns"):
            setattr(cfg, name, int(getattr(config, name)))
        cfg.enable_mask = 1 if config.enable_mask else 0
        cfg.alloc.alloc_fn, cfg.alloc.free_fn, cfg.alloc.context = config.alloc.alloc_fn or None, config.alloc.free_fn or None, config.alloc.context or None
        g = ctypes.c_void_p()
        _lib.check(lib.ncclEpCreateGroup(ctypes.byref(g), inner.handle, ctypes.byref(cfg)), "ncclEpCreateGroup", lib)
        return cls(g, lib)

    def _check_valid(self, operation):
        if not self._ptr:
            raise RuntimeError("%s on a group that was destroyed" % operation)

    @property
    def ptr(self):
        return self._ptr.value if self._ptr else 0

    def create_handle(self, layout, topk_idx, *, layout_info=None, config=None, stream=None):
        self._check_valid("create_handle")
        h = ctypes.c_void_p()
        li = layout_info._struct() if layout_info is not None else None
        hc = None
        if config is not None:
            hc = _HandleCfg(ctypes.sizeof(_HandleCfg), _ep.EP_MAGIC, int(config.dispatch_output_per_expert_alignment))
        _lib.check(self._lib.ncclEpCreateHandle(ctypes.byref(h), self._ptr, int(layout), _p(topk_idx), ctypes.byref(li) if li is not None else None,
                                                ctypes.byref(hc) if hc is not None else None, _stream_ptr(stream)), "ncclEpCreateHandle", self._lib)
        handle = Handle(h, self._lib)
        handle._keep = (topk_idx, layout_info, li)
        return handle

    def destroy(self):
        if self._ptr:
            self._lib.ncclEpGroupDestroy(self._ptr)
            self._ptr = None

    def __repr__(self):
        return "Group(ptr=0x%x)" % self.ptr
