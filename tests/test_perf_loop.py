"""The loop of collective calls that the timing harness runs outside the interpreter (tools/perf_loop.c), driven here on host
ranks: every call shape it knows reaches the library with the right arguments."""
import ctypes
import os

import numpy as np

from mp_util import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}


def _rank(rank, nranks, uid):
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    L = comm.lib
    loop = ctypes.CDLL(os.path.join(ROOT, "nccl_b200", "lib", "libperf_loop.so")).perfLoop
    loop.restype = ctypes.c_int
    loop.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                     ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]

    def fns(*names):
        return (ctypes.c_void_p * len(names))(*[ctypes.cast(getattr(L, n), ctypes.c_void_p).value for n in names])

    n, FP32 = nranks, 7
    out = {}
    x = np.full(64, rank + 1, dtype=np.float32)
    y = np.zeros(64, dtype=np.float32)
    nxt, prv = (rank + 1) % n, (rank - 1) % n
    args = lambda s, r, count: (s.ctypes.data, r.ctypes.data, count, FP32, 0, 0, nxt, prv, comm.handle, None)  # noqa: E731
    assert loop(0, fns("ncclAllReduce"), *args(x, y, 64), 3) == 0
    out["all_reduce"] = float(y[0])
    g = np.zeros(64 * n, dtype=np.float32)
    assert loop(1, fns("ncclAllGather"), *args(x, g, 64), 2) == 0
    out["all_gather"] = [float(g[i * 64]) for i in range(n)]
    rs = np.zeros(64 // n, dtype=np.float32)
    assert loop(0, fns("ncclReduceScatter"), *args(x, rs, 64 // n), 2) == 0
    out["reduce_scatter"] = float(rs[0])
    b = np.zeros(64, dtype=np.float32)
    assert loop(2, fns("ncclBroadcast"), *args(x, b, 64), 2) == 0
    out["broadcast"] = float(b[0])
    rd = np.zeros(64, dtype=np.float32)
    assert loop(3, fns("ncclReduce"), *args(x, rd, 64), 2) == 0
    out["reduce"] = float(rd[0])
    sr = np.zeros(64, dtype=np.float32)
    assert loop(4, fns("ncclGroupStart", "ncclSend", "ncclRecv", "ncclGroupEnd"), *args(x, sr, 64), 2) == 0
    out["sendrecv"] = float(sr[0])
    assert loop(9, fns("ncclAllReduce"), *args(x, y, 64), 1) == -1
    comm.destroy()
    return out


def test_every_call_shape_of_the_loop():
    n = 2
    res = run_ranks(_rank, n, env=BASE)
    total = n * (n + 1) / 2
    for r in range(n):
        o = res[r]
        assert o["all_reduce"] == total and o["reduce_scatter"] == total and o["broadcast"] == 1.0
        assert o["all_gather"] == [1.0, 2.0]
        assert o["reduce"] == (total if r == 0 else 0.0)
        assert o["sendrecv"] == (r - 1) % n + 1


def _harness_rank(rank, nranks, uid, python_loop):
    """Harness.calls without the CUDA set-up of its constructor: host buffers and a host communicator."""
    if python_loop:
        os.environ["NCCL_B200_PERF_PYTHON_LOOP"] = "1"
    from nccl_b200 import Communicator
    from nccl_b200.utils.perf import Harness
    comm = Communicator(nranks, rank, uid)
    h = object.__new__(Harness)
    h.lib, h.comm, h.n, h.rank = comm.lib, comm.handle, nranks, rank
    x = np.full(256, rank + 1, dtype=np.float32)
    y = np.zeros(256 * nranks, dtype=np.float32)
    h.send_ptr, h.recv_ptr = x.ctypes.data, y.ctypes.data
    out = {}
    for coll, nbytes in (("all_reduce", 1024), ("all_gather", 1024 * nranks), ("reduce_scatter", 1024), ("all_to_all", 1024), ("broadcast", 1024), ("sendrecv", 1024)):
        y[:] = 0
        assert h.calls(coll, nbytes, 7, None, 3) == 0
        out[coll] = [float(v) for v in y[:: 256 // nranks][: 2 * nranks]]
    out["native"] = h._native_loop() is not None
    comm.destroy()
    return out


def test_the_harness_issues_the_same_calls_through_either_loop():
    a = run_ranks(_harness_rank, 2, args=(False,), env=BASE)
    b = run_ranks(_harness_rank, 2, args=(True,), env=BASE)
    assert a[0]["native"] and not b[0]["native"]
    for r in range(2):
        for coll in ("all_reduce", "all_gather", "reduce_scatter", "all_to_all", "broadcast", "sendrecv"):
            assert a[r][coll] == b[r][coll], (r, coll, a[r][coll], b[r][coll])
    assert a[0]["all_reduce"][0] == 3.0 and a[1]["sendrecv"][0] == 1.0
