"""Failure detection on the host (no GPU involved, nothing faults): a rank that never joins, a
stranger on the rendezvous port, a peer that leaves between steps, and an abort from another
thread while a collective is blocked."""
import os
import socket
import struct
import threading
import time

import numpy as np
import pytest

from mp_util import run_ranks

ENV = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}


def _init_only(rank, nranks, uid, announced):
    from nccl_b200 import Communicator, _lib
    t0 = time.time()
    try:
        Communicator(announced, rank, uid)
    except _lib.NcclError as e:
        return "error", e.code, time.time() - t0
    return "ok", 0, time.time() - t0


def test_rank_that_never_joins_times_out():
    # three ranks are announced, two show up: the rendezvous gives up after the socket time-out
    env = dict(ENV, NCCL_B200_SOCKET_TIMEOUT_MS="1500")
    res = run_ranks(_init_only, 2, args=(3,), env=env, timeout=60)
    for r in range(2):
        status, code, dt = res[r]
        assert status == "error" and code in (2, 3, 6, 8), res[r]   # ncclTimeout (8) is the expected code
        assert dt < 30


def _stranger_then_allreduce(rank, nranks, uid):
    from nccl_b200 import Communicator
    if rank == 0:
        # a connection that does not speak the protocol (wrong magic) must be dropped by the root
        fam, port = struct.unpack_from("<HH", uid, 8)
        port = socket.ntohs(port)
        ip = socket.inet_ntoa(uid[12:16])
        s = socket.create_connection((ip, port), timeout=5)
        s.sendall(b"\x01\x02\x03\x04\x05\x06\x07\x08" + struct.pack("<i", 1) + b"junk" * 8)
        time.sleep(0.2)
        s.close()
    comm = Communicator(nranks, rank, uid)
    x = np.full(64, rank + 1.0, dtype=np.float32)
    comm.all_reduce(x)
    comm.destroy()
    return float(x[0])


def test_stranger_on_the_rendezvous_port_is_ignored():
    res = run_ranks(_stranger_then_allreduce, 2, env=ENV, timeout=60)
    assert res[0] == 3.0 and res[1] == 3.0


def _peer_leaves(rank, nranks, uid):
    from nccl_b200 import Communicator, _lib
    comm = Communicator(nranks, rank, uid)
    x = np.ones(1 << 14, dtype=np.float32)
    comm.all_reduce(x)          # one good step
    if rank == 1:
        os._exit(0)             # leaves between steps; its sockets close
    t0 = time.time()
    try:
        comm.all_reduce(x)
        return "ok", 0, time.time() - t0
    except _lib.NcclError as e:
        return "error", e.code, time.time() - t0


def test_peer_that_leaves_turns_into_an_error():
    res = run_ranks(_peer_leaves, 2, env=dict(ENV, NCCL_B200_SOCKET_TIMEOUT_MS="3000"), timeout=60, may_exit=(1,))
    status, code, dt = res[0]
    assert status == "error" and code in (2, 6), res[0]     # system / remote error, not a hang
    assert dt < 20


def _abort_unblocks(rank, nranks, uid):
    from nccl_b200 import Communicator, _lib
    comm = Communicator(nranks, rank, uid)
    x = np.ones(1 << 14, dtype=np.float32)
    comm.all_reduce(x)
    if rank == 1:
        time.sleep(3.0)         # never enters the second collective in time
        return "late", 0, 0.0
    handle = comm.handle
    lib = comm.lib

    def aborter():
        time.sleep(0.5)
        lib.ncclCommAbort(handle)

    th = threading.Thread(target=aborter)
    th.start()
    t0 = time.time()
    try:
        comm.all_reduce(x)
        out = ("ok", 0, time.time() - t0)
    except _lib.NcclError as e:
        out = ("error", e.code, time.time() - t0)
    th.join()
    comm.handle = None
    return out


def test_abort_from_another_thread_unblocks_a_collective():
    res = run_ranks(_abort_unblocks, 2, env=ENV, timeout=60)
    status, code, dt = res[0]
    assert status == "error", res[0]
    assert dt < 2.5, "the blocked collective returned only after %.1f s" % dt


def _two_threads_rank(rank, nranks, uid, fatal):
    import threading
    import time
    import numpy as np
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    x = np.full(1 << 16, rank + 1.0, dtype=np.float32)
    second = {}
    if rank == 1:
        time.sleep(1.0)                      # keeps rank 0 inside its all-reduce for a second
        comm.all_reduce(x)
    else:
        def late():
            y = np.ones(16, dtype=np.float32)
            try:
                time.sleep(0.3)
                if fatal:
                    comm.all_reduce(y)       # refused: another thread is inside a call on this communicator
                second["rc"] = "ok"
            except Exception as e:           # noqa: BLE001
                second["rc"] = str(e)
        t = threading.Thread(target=late)
        t.start()
        comm.all_reduce(x)
        t.join()
    comm.destroy()
    return float(x[0]), second.get("rc")


def test_two_threads_on_one_communicator_are_detected():
    """Calls on one communicator must be serialised: the later of two concurrent calls fails with ncclInvalidUsage
    (NCCL_LAUNCH_RACE_FATAL=1, the default) and the first one completes normally."""
    res = run_ranks(_two_threads_rank, 2, args=(True,), env=ENV, timeout=120)
    assert res[0][0] == 3.0 and res[1][0] == 3.0
    assert "ncclInvalidUsage" in res[0][1] and "two threads" in res[0][1], res[0][1]
