"""Public API semantics on CPU ranks: argument checks, error strings, communicator queries, splits
(colour, key, no-colour), shrink, pre-multiplied sums, gather / scatter, scalable init with several
roots, and communicator creation inside a group."""
import ctypes

import numpy as np
import pytest

from mp_util import run_ranks

ENV = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}


def _queries(rank, nranks, uid):
    from nccl_b200 import Communicator, _lib, version
    from nccl_b200.core import FP32
    comm = Communicator(nranks, rank, uid)
    lib = comm.lib
    n, r, dev = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    assert lib.ncclCommCount(comm.handle, ctypes.byref(n)) == 0 and n.value == nranks
    assert lib.ncclCommUserRank(comm.handle, ctypes.byref(r)) == 0 and r.value == rank
    lib.ncclGetErrorString.restype = ctypes.c_char_p
    assert b"invalid argument" in lib.ncclGetErrorString(4).lower()
    out = {"version": version(lib)}
    x = np.ones(8, dtype=np.float32)
    # argument checks: bad root, bad type, null communicator
    out["bad_root"] = lib.ncclBroadcast(x.ctypes.data, x.ctypes.data, 8, FP32, nranks + 3, comm.handle, None)
    out["bad_type"] = lib.ncclAllReduce(x.ctypes.data, x.ctypes.data, 8, 99, 0, comm.handle, None)
    out["null_comm"] = lib.ncclAllReduce(x.ctypes.data, x.ctypes.data, 8, FP32, 0, None, None)
    lib.ncclGetLastError.restype = ctypes.c_char_p
    out["last_error"] = lib.ncclGetLastError(comm.handle).decode()
    assert comm.async_error() == 0
    # zero-count collectives are no-ops
    assert lib.ncclAllReduce(x.ctypes.data, x.ctypes.data, 0, FP32, 0, comm.handle, None) == 0
    comm.destroy()
    return out


def test_queries_and_argument_checks():
    res = run_ranks(_queries, 2, env=ENV)
    for r in range(2):
        o = res[r]
        assert o["version"] >= 23000
        assert o["bad_root"] == 4 and o["bad_type"] == 4 and o["null_comm"] == 4   # ncclInvalidArgument
        assert o["last_error"]


def _splits(rank, nranks, uid):
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    out = {}
    # colour = parity, key reverses the order inside each half
    sub = comm.split(rank % 2, key=-rank)
    out["sub"] = (sub.nranks, sub.rank)
    x = np.full(4, float(rank), dtype=np.float64)
    sub.all_reduce(x)
    out["sub_sum"] = float(x[0])
    sub.destroy()
    # ranks with no colour get no communicator
    none = comm.split(-1 if rank == 0 else 0)
    out["nocolor"] = None if none is None or none.handle is None or not none.handle else (none.nranks, none.rank)
    if out["nocolor"] is not None:
        y = np.ones(2, dtype=np.float32)
        none.all_reduce(y)
        out["nocolor_sum"] = float(y[0])
        none.destroy()
    # shrink: drop the last rank
    if rank != nranks - 1:
        sh = comm.shrink([nranks - 1])
        z = np.ones(3, dtype=np.float32)
        sh.all_reduce(z)
        out["shrunk"] = (sh.nranks, float(z[0]))
        sh.destroy()
    comm.destroy()
    return out


def test_split_nocolor_and_shrink():
    n = 4
    res = run_ranks(_splits, n, env=ENV, timeout=120)
    for r in range(n):
        o = res[r]
        members = [q for q in range(n) if q % 2 == r % 2]
        assert o["sub"][0] == len(members)
        assert o["sub"][1] == sorted(members, reverse=True).index(r)
        assert o["sub_sum"] == float(sum(members))
        if r == 0:
            assert o["nocolor"] is None
        else:
            assert o["nocolor"][0] == n - 1 and o["nocolor_sum"] == n - 1
        if r != n - 1:
            assert o["shrunk"] == (n - 1, float(n - 1))


def _premul_gather(rank, nranks, uid):
    from nccl_b200 import Communicator
    from nccl_b200.core import FP32
    comm = Communicator(nranks, rank, uid)
    out = {}
    op = comm.premul_sum(0.5, FP32)
    x = np.full(6, float(rank + 1), dtype=np.float32)
    y = np.zeros_like(x)
    comm.all_reduce(x, y, op=op)
    comm.destroy_op(op)
    out["premul"] = float(y[0])
    g = np.zeros(nranks * 3, dtype=np.int32)
    comm.gather(np.full(3, rank, dtype=np.int32), g, root=1)
    out["gather"] = g.tolist()
    s = np.zeros(2, dtype=np.int32)
    comm.scatter(np.arange(2 * nranks, dtype=np.int32) if rank == 0 else np.zeros(2 * nranks, dtype=np.int32), s, root=0)
    out["scatter"] = s.tolist()
    comm.destroy()
    return out


def test_premultiplied_sum_gather_scatter():
    n = 3
    res = run_ranks(_premul_gather, n, env=ENV)
    for r in range(n):
        assert res[r]["premul"] == 0.5 * n * (n + 1) / 2
        assert res[r]["scatter"] == [2 * r, 2 * r + 1]
    assert res[1]["gather"] == [q for q in range(n) for _ in range(3)]


def _scalable(rank, nranks, uids):
    """ncclCommInitRankScalable with two roots: every rank knows both unique ids."""
    from nccl_b200 import Communicator, _lib
    lib = _lib.load()
    ids = (_lib.ncclUniqueId * 2)()
    for i in range(2):
        ctypes.memmove(ctypes.byref(ids[i]), uids[i * 128:(i + 1) * 128], 128)
    h = _lib.ncclComm_t()
    lib.ncclCommInitRankScalable.argtypes = [ctypes.POINTER(_lib.ncclComm_t), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_lib.ncclUniqueId), ctypes.c_void_p]
    _lib.check(lib.ncclCommInitRankScalable(ctypes.byref(h), nranks, rank, 2, ids, None), "ncclCommInitRankScalable", lib)
    comm = Communicator(nranks, rank, None, lib=lib, _handle=h)
    x = np.full(5, float(rank), dtype=np.float32)
    comm.all_reduce(x)
    comm.destroy()
    return float(x[0])


def test_scalable_init_with_two_roots():
    from nccl_b200 import get_unique_id
    n = 5
    res = run_ranks(_scalable, n, env=ENV, make_uid=lambda: get_unique_id() + get_unique_id(), timeout=120)
    for r in range(n):
        assert res[r] == float(sum(range(n)))


def _host_staged_rank(rank, nranks, uid):
    import ctypes
    import numpy as np
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    buf = np.ones(16, dtype=np.float32)
    fn = comm.lib.ncclAllReduceFromHost
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    p = buf.ctypes.data
    rc = fn(p, p, p, p, 16, 7, 0, comm.handle, None, 0)
    comm.all_reduce(buf.copy(), buf)   # the communicator is still usable
    comm.destroy()
    return rc


def test_host_staged_allreduce_needs_a_gpu_communicator():
    """ncclAllReduceFromHost stages through device memory: a host-memory communicator refuses it (its own
    ncclAllReduce already works on host buffers)."""
    from mp_util import run_ranks
    res = run_ranks(_host_staged_rank, 2, env={"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"})
    assert res[0] == 5 and res[1] == 5   # ncclInvalidUsage
