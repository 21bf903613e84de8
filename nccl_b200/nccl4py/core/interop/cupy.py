"""CuPy helpers with the shapes of the PyTorch ones: ``empty`` gives an array in memory of ncclMemAlloc, ``resolve_array``
describes an array for the C calls. CuPy is optional; both raise ModuleNotFoundError without it.

Reference parity: bindings/nccl4py/nccl/core/interop/cupy.py (empty, resolve_array).
"""
import numpy as np

from .... import core as _core

try:
    import cupy
    _cupy_enabled = True
except ImportError:
    _cupy_enabled = False

__all__ = ["empty", "resolve_array"]

_TYPES = {"int8": _core.INT8, "uint8": _core.UINT8, "int32": _core.INT32, "uint32": _core.UINT32, "int64": _core.INT64, "uint64": _core.UINT64,
          "float16": _core.FP16, "float32": _core.FP32, "float64": _core.FP64}


def empty(shape, dtype=np.float32, order="C"):
    if not _cupy_enabled:
        raise ModuleNotFoundError("CuPy is not installed")
    if order not in ("C", "F"):
        raise ValueError("order must be 'C' or 'F', got %r" % (order,))
    shape = (shape,) if isinstance(shape, int) else tuple(shape)
    dtype = np.dtype(dtype)
    nbytes = max(int(np.prod(shape, dtype=np.int64)) * dtype.itemsize, 1)
    ptr = _core.mem_alloc(nbytes)

    class _Owner:
        def __del__(self, ptr=ptr):
            try:
                _core.mem_free(ptr)
            except Exception:
                pass

    mem = cupy.cuda.UnownedMemory(ptr, nbytes, _Owner())
    return cupy.ndarray(shape, dtype=dtype, memptr=cupy.cuda.MemoryPointer(mem, 0), order=order)


def resolve_array(array):
    if not _cupy_enabled:
        raise ModuleNotFoundError("CuPy is not installed")
    if not (array.flags.c_contiguous or array.flags.f_contiguous):
        raise ValueError("array must be dense (row- or column-major)")
    name = np.dtype(array.dtype).name
    if name not in _TYPES:
        raise ValueError("no NCCL data type for %s" % name)
    return int(array.data.ptr), int(array.size), _TYPES[name], int(array.device.id)
