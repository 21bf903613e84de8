"""The call shapes of the reference's Python package (``nccl.core``) over this library.

Programs written against the reference's bindings keep their spelling::

    import nccl_b200.nccl4py.core as nccl
    uid = nccl.get_unique_id()                       # rank 0, then broadcast the bytes
    comm = nccl.Communicator.init(nranks, rank, uid)
    comm.allreduce(x, y, nccl.SUM, stream=s)
    with nccl.group():
        comm.send(a, peer=1); comm.recv(b, peer=1)

``nccl_b200.nccl4py.ep`` has the shapes of the reference's ``nccl.ep`` (groups, handles, tensor descriptors) and is imported on demand.

Reference parity: bindings/nccl4py/nccl/core/{communicator,group,memory,utils,constants}.py, bindings/nccl4py/nccl/ep/.
"""
from . import core  # noqa: F401
from ._show_versions import LibraryInfo, VersionInfo, get_version, show_versions  # noqa: F401
