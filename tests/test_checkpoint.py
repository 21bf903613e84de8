"""Checkpoint support on CPU ranks: a communicator is taken down, its record travels through a
byte string (as it would inside a process image), and an equivalent communicator is built from it
with a fresh unique id."""
import ctypes
import os
import time

import numpy as np

from mp_util import run_ranks


def _rank(rank, nranks, uid, tmp):
    from nccl_b200 import Communicator, _lib, get_unique_id
    from nccl_b200.core import unique_id_from_bytes
    lib = _lib.load()
    P = ctypes.c_void_p
    lib.ncclCommCheckpointPrepare.argtypes = [P, ctypes.POINTER(P)]
    lib.ncclCommCheckpointSave.argtypes = [P, P, ctypes.POINTER(ctypes.c_size_t)]
    lib.ncclCommCheckpointLoad.argtypes = [P, ctypes.c_size_t, ctypes.POINTER(P)]
    lib.ncclCommCheckpointRestore.argtypes = [P, _lib.ncclUniqueId, ctypes.POINTER(P), P, ctypes.c_int]
    lib.ncclCommCheckpointFree.argtypes = [P]
    comm = Communicator(nranks, rank, uid)
    x = np.full(1000, rank + 1.0, dtype=np.float32)
    comm.all_reduce(x)
    first = float(x[0])
    # take the communicator down and serialise its record
    st = P()
    _lib.check(lib.ncclCommCheckpointPrepare(comm.handle, ctypes.byref(st)), "ncclCommCheckpointPrepare", lib)
    comm.handle = None
    size = ctypes.c_size_t(0)
    _lib.check(lib.ncclCommCheckpointSave(st, None, ctypes.byref(size)), "ncclCommCheckpointSave", lib)
    buf = ctypes.create_string_buffer(size.value)
    _lib.check(lib.ncclCommCheckpointSave(st, buf, ctypes.byref(size)), "ncclCommCheckpointSave", lib)
    lib.ncclCommCheckpointFree(st)
    record = bytes(buf.raw[:size.value])
    # ... the process image would be written and restored here ...
    # a fresh unique id reaches every rank the way it does at start-up (here: a file)
    path = os.path.join(tmp, "uid")
    if rank == 0:
        raw = get_unique_id(lib)
        with open(path + ".tmp", "wb") as f:
            f.write(raw)
        os.rename(path + ".tmp", path)
    deadline = time.time() + 30
    while not os.path.exists(path) and time.time() < deadline:
        time.sleep(0.02)
    raw = open(path, "rb").read()
    st2 = P()
    _lib.check(lib.ncclCommCheckpointLoad(record, len(record), ctypes.byref(st2)), "ncclCommCheckpointLoad", lib)
    h = P()
    _lib.check(lib.ncclCommCheckpointRestore(st2, unique_id_from_bytes(raw), ctypes.byref(h), None, 0), "ncclCommCheckpointRestore", lib)
    lib.ncclCommCheckpointFree(st2)
    comm2 = Communicator(nranks, rank, None, lib=lib, _handle=h)
    y = np.full(1000, 10.0 * (rank + 1), dtype=np.float32)
    comm2.all_reduce(y)
    out = (first, float(y[0]), comm2.nranks, comm2.rank)
    comm2.destroy()
    return out


def test_prepare_save_load_restore(tmp_path):
    n = 3
    res = run_ranks(_rank, n, args=(str(tmp_path),), env={"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}, timeout=120)
    for r in range(n):
        assert res[r] == (6.0, 60.0, n, r)


def _process_wide_rank(rank, nranks, uid):
    from nccl_b200 import Communicator, _lib
    comm = Communicator(nranks, rank, uid)
    lib = comm.lib
    ck, nv = ctypes.c_int(), ctypes.c_int()
    assert lib.ncclCheckpointGetVersion(ctypes.byref(ck), ctypes.byref(nv)) == 0
    x = np.full(100, rank + 1.0, dtype=np.float32)
    comm.all_reduce(x)
    _lib.check(lib.ncclCheckpointPrepare(), "ncclCheckpointPrepare", lib)
    _lib.check(lib.ncclCheckpointRestore(), "ncclCheckpointRestore", lib)
    y = np.full(100, rank + 1.0, dtype=np.float32)
    comm.all_reduce(y)     # the same handle keeps working
    comm.destroy()
    _lib.check(lib.ncclCheckpointPrepare(), "ncclCheckpointPrepare", lib)   # no communicator left: nothing to do
    _lib.check(lib.ncclCheckpointRestore(), "ncclCheckpointRestore", lib)
    return ck.value, nv.value, float(x[0]), float(y[0])


def test_process_wide_prepare_restore():
    """The reference's argument-less entry points: host-memory communicators hold nothing on a GPU, so the calls
    succeed and leave the communicator usable."""
    res = run_ranks(_process_wide_rank, 2, env={"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}, timeout=120)
    for r in range(2):
        assert res[r] == (1, 23007, 3.0, 3.0)
