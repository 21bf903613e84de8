"""PyTorch helpers: ``empty`` gives a tensor whose memory comes from ncclMemAlloc (shareable, registrable as a symmetric
window, multicast-bindable) and is returned to the library when the tensor is collected; ``resolve_tensor`` describes a tensor
for the C calls.

Reference parity: bindings/nccl4py/nccl/core/interop/torch.py (empty, resolve_tensor).
"""
import weakref

from .... import core as _core

try:
    import torch
    _torch_enabled = True
except ImportError:   # pragma: no cover
    _torch_enabled = False

__all__ = ["empty", "resolve_tensor"]


class _Allocation:
    """Owns one ncclMemAlloc range; freed when the last tensor over it is gone."""

    def __init__(self, nbytes, device):
        self.device = device
        with torch.cuda.device(device):
            self.ptr = _core.mem_alloc(max(int(nbytes), 1))
        self.__cuda_array_interface__ = {"shape": (max(int(nbytes), 1),), "typestr": "|u1", "data": (self.ptr, False), "version": 2}
        self._finalizer = weakref.finalize(self, _free, self.ptr, device)


def _free(ptr, device):
    try:
        with torch.cuda.device(device):
            torch.cuda.synchronize()
            _core.mem_free(ptr)
    except Exception:   # interpreter shutdown: the driver reclaims the memory
        pass


def _parse_device(device):
    if device is None:
        return torch.cuda.current_device()
    if isinstance(device, int):
        return device
    d = torch.device(device)
    if d.type != "cuda":
        raise ValueError("device must be a CUDA device, got %r" % (device,))
    return torch.cuda.current_device() if d.index is None else d.index


def empty(*size, dtype=None, device=None, morder="C"):
    """An uninitialised tensor in memory of the library's allocator. ``morder`` "F" gives column-major strides."""
    if not _torch_enabled:
        raise ModuleNotFoundError("PyTorch is not installed")
    if morder not in ("C", "F"):
        raise ValueError("morder must be 'C' or 'F', got %r" % (morder,))
    shape = tuple(size[0]) if len(size) == 1 and isinstance(size[0], (tuple, list)) else tuple(int(s) for s in size)
    dtype = dtype or torch.get_default_dtype()
    dev = _parse_device(device)
    numel = 1
    for s in shape:
        numel *= s
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    alloc = _Allocation(nbytes, dev)
    flat = torch.as_tensor(alloc, device="cuda:%d" % dev)[:nbytes].view(dtype)   # the tensor keeps `alloc` alive through the array interface
    if morder == "C" or len(shape) < 2:
        return flat.view(shape) if numel else flat.new_empty(shape)
    strides, acc = [], 1
    for s in shape:
        strides.append(acc)
        acc *= s
    return flat.as_strided(shape, strides)


def resolve_tensor(tensor):
    """``(data pointer, element count, NCCL data type, device index)`` of a contiguous CUDA tensor."""
    if not _torch_enabled:
        raise ModuleNotFoundError("PyTorch is not installed")
    if not tensor.is_contiguous() and not tensor.t().is_contiguous():
        raise ValueError("tensor must be dense (row- or column-major)")
    ptr, n, dt, _ = _core.describe(tensor)
    return ptr, n, dt, tensor.device.index if tensor.is_cuda else -1
