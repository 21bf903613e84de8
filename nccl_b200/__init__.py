"""B200-native collective communication library with the NCCL host API.

``nccl_b200.core`` wraps the C API (communicators, collectives, windows); ``nccl_b200.ops`` has
symmetric tensors and the fused tensor-parallel / expert-parallel operators; ``nccl_b200.parallel``
has the data-parallel, FSDP, pipeline and context-parallel drivers; ``nccl_b200.models`` the Llama-shaped model used by the benches.
"""
from . import _lib  # noqa: F401
from .core import (AVG, MAX, MIN, PROD, SUM, Communicator, get_unique_id, group, mem_alloc, mem_free,  # noqa: F401
                   version)

__all__ = ["Communicator", "get_unique_id", "group", "mem_alloc", "mem_free", "version", "SUM", "PROD", "MAX", "MIN", "AVG"]
