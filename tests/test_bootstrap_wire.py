"""Bootstrap wire compatibility with the reference library.

CPU: the rendezvous root is the reference library's own root thread (created by its
ncclGetUniqueId in the parent process); ranks of this library check in with it, receive their ring
neighbour from it and complete an all-reduce. GPU (two devices): the roles are swapped: ranks of the
reference library rendezvous through this library's root.
Skipped when the reference build (baseline/_ref) is not present."""
import ctypes
import os

import numpy as np
import pytest

from mp_util import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "baseline", "_ref", "build", "lib", "libnccl.so.2")


class _Uid(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_char * 128)]


def _our_rank(rank, nranks, uid):
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    x = np.full(4096, rank + 1.0, dtype=np.float32)
    y = np.zeros_like(x)
    comm.all_reduce(x, y)
    comm.destroy()
    return float(y[0]), float(y[-1])


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="reference build not present")
def test_our_ranks_through_reference_root():
    os.environ["NCCL_SOCKET_IFNAME"] = "lo"
    ref = ctypes.CDLL(REF_LIB)

    def make_uid():
        u = _Uid()
        assert ref.ncclGetUniqueId(ctypes.byref(u)) == 0
        return ctypes.string_at(ctypes.byref(u), 128)

    n = 3
    res = run_ranks(_our_rank, n, env={"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}, make_uid=make_uid)
    for r in range(n):
        assert res[r] == (n * (n + 1) / 2, n * (n + 1) / 2)


def _ref_rank(rank, nranks, uid):
    import ctypes
    import torch
    torch.cuda.set_device(rank)
    lib = ctypes.CDLL(REF_LIB)
    comm = ctypes.c_void_p()
    u = _Uid()
    ctypes.memmove(ctypes.byref(u), uid, 128)
    lib.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, _Uid, ctypes.c_int]
    assert lib.ncclCommInitRank(ctypes.byref(comm), nranks, u, rank) == 0
    x = torch.full((1 << 16,), float(rank + 1), device="cuda")
    lib.ncclAllReduce.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    assert lib.ncclAllReduce(x.data_ptr(), x.data_ptr(), x.numel(), 7, 0, comm, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    out = float(x[0])
    lib.ncclCommDestroy.argtypes = [ctypes.c_void_p]
    lib.ncclCommDestroy(comm)
    return out


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="reference build not present")
def test_reference_ranks_through_our_root():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = run_ranks(_ref_rank, 2, env={"NCCL_SOCKET_IFNAME": "lo"})   # the unique id comes from this library's root thread
    assert res[0] == 3.0 and res[1] == 3.0
