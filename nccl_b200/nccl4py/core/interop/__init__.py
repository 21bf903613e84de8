"""Framework helpers: tensors and arrays backed by the library's allocator (``torch``, ``cupy``), imported on demand.

Reference parity: bindings/nccl4py/nccl/core/interop/.
"""
