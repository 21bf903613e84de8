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
    lib.ncclCheckpointPrepare.argtypes = [P, ctypes.POINTER(P)]
    lib.ncclCheckpointSave.argtypes = [P, P, ctypes.POINTER(ctypes.c_size_t)]
    lib.ncclCheckpointLoad.argtypes = [P, ctypes.c_size_t, ctypes.POINTER(P)]
    lib.ncclCheckpointRestore.argtypes = [P, _lib.ncclUniqueId, ctypes.POINTER(P), P, ctypes.c_int]
    lib.ncclCheckpointFree.argtypes = [P]
    comm = Communicator(nranks, rank, uid)
    x = np.full(1000, rank + 1.0, dtype=np.float32)
    comm.all_reduce(x)
    first = float(x[0])
    # take the communicator down and serialise its record
    st = P()
    _lib.check(lib.ncclCheckpointPrepare(comm.handle, ctypes.byref(st)), "ncclCheckpointPrepare", lib)
    comm.handle = None
    size = ctypes.c_size_t(0)
    _lib.check(lib.ncclCheckpointSave(st, None, ctypes.byref(size)), "ncclCheckpointSave", lib)
    buf = ctypes.create_string_buffer(size.value)
    _lib.check(lib.ncclCheckpointSave(st, buf, ctypes.byref(size)), "ncclCheckpointSave", lib)
    lib.ncclCheckpointFree(st)
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
    _lib.check(lib.ncclCheckpointLoad(record, len(record), ctypes.byref(st2)), "ncclCheckpointLoad", lib)
    h = P()
    _lib.check(lib.ncclCheckpointRestore(st2, unique_id_from_bytes(raw), ctypes.byref(h), None, 0), "ncclCheckpointRestore", lib)
    lib.ncclCheckpointFree(st2)
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
