"""InfiniBand / RoCE backend on CPU ranks against a stand-in for libibverbs (tests/data/fake_ibverbs.cc: queue pairs
whose traffic travels over UNIX sockets, with key, bounds and state checks). The host collectives of several processes
go through the backend and the proxy thread; the stand-in counts protocol violations."""
import os
import subprocess

import numpy as np
import pytest

from mp_util import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo", "NCCL_B200_HOST_NET": "1"}


@pytest.fixture(scope="module")
def fake_lib(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("fakeib") / "libfakeibverbs.so")
    subprocess.run(["g++", "-std=c++17", "-O1", "-shared", "-fPIC", "-I" + os.path.join(ROOT, "src", "transport"),
                    os.path.join(ROOT, "tests", "data", "fake_ibverbs.cc"), "-o", out, "-pthread"], check=True)
    return out


def _rank(rank, nranks, uid, sizes):
    import ctypes
    from nccl_b200 import Communicator, group
    comm = Communicator(nranks, rank, uid)
    out = []
    for n in sizes:
        x = (np.arange(n, dtype=np.float32) % 251) + rank
        y = np.zeros_like(x)
        comm.all_reduce(x, y)
        ref = (np.arange(n, dtype=np.float32) % 251) * nranks + nranks * (nranks - 1) / 2
        out.append(bool(np.array_equal(y, ref)))
    peer, src = (rank + 1) % nranks, (rank - 1) % nranks
    for n in sizes:
        s = np.full(n, rank + 1, dtype=np.float32)
        r = np.zeros(n, dtype=np.float32)
        with group():
            comm.send(s, peer)
            comm.recv(r, src)
        out.append(bool((r == src + 1).all()))
    comm.destroy()
    errs = ctypes.CDLL(os.environ["NCCL_B200_IBV_LIB"]).fake_ib_errors()
    return out, errs


@pytest.mark.parametrize("link", ["ETH", "IB"])
def test_host_collectives_over_the_verbs_backend(fake_lib, tmp_path, link):
    env = dict(BASE, NCCL_NET="IB", NCCL_B200_IBV_LIB=fake_lib, FAKE_IB_LINK=link, NCCL_DEBUG="INFO", NCCL_DEBUG_SUBSYS="NET,INIT",
               NCCL_DEBUG_FILE=str(tmp_path / "log.%p"))
    # 1 element (inline), 1000 floats (eager through the staging ring), 64 Ki and 1 Mi floats (credits + RDMA writes, several slices)
    res = run_ranks(_rank, 3, args=([1, 1000, 1 << 16, 1 << 20],), env=env, timeout=300)
    for r in range(3):
        ok, errs = res[r]
        assert all(ok), (r, ok)
        assert errs == 0
    text = "".join(open(tmp_path / f).read() for f in os.listdir(tmp_path))
    assert "network backend: built-in IB, 2 device(s)" in text
    assert ("RoCE" if link == "ETH" else "InfiniBand") in text


def test_device_filter_and_fallback_to_sockets(fake_lib, tmp_path):
    env = dict(BASE, NCCL_B200_IBV_LIB=fake_lib, NCCL_IB_HCA="^fakeib", NCCL_DEBUG="INFO", NCCL_DEBUG_SUBSYS="NET,INIT", NCCL_DEBUG_FILE=str(tmp_path / "log.%p"))
    res = run_ranks(_rank, 2, args=([1 << 12],), env=env, timeout=200)
    assert all(all(res[r][0]) for r in range(2))
    text = "".join(open(tmp_path / f).read() for f in os.listdir(tmp_path))
    assert "built-in IB" not in text


def test_one_device_selected_by_name(fake_lib, tmp_path):
    env = dict(BASE, NCCL_B200_IBV_LIB=fake_lib, NCCL_IB_HCA="=fakeib1:1", NCCL_DEBUG="INFO", NCCL_DEBUG_SUBSYS="NET,INIT", NCCL_DEBUG_FILE=str(tmp_path / "log.%p"),
               NCCL_B200_IB_EAGER_BYTES="256", NCCL_IB_USE_INLINE="0")
    res = run_ranks(_rank, 2, args=([3, 64, 100, 5000],), env=env, timeout=200)
    for r in range(2):
        assert all(res[r][0]) and res[r][1] == 0
    text = "".join(open(tmp_path / f).read() for f in os.listdir(tmp_path))
    assert "built-in IB, 1 device(s)" in text and "fakeib1:1" in text and "fakeib0" not in text


def _many_rank(rank, nranks, uid):
    import ctypes
    from nccl_b200 import Communicator, group
    comm = Communicator(nranks, rank, uid)
    peer, src = (rank + 1) % nranks, (rank - 1) % nranks
    sizes = [1, 3000, 17, 40000, 2048, 2049, 70000, 5] * 12      # 96 messages per direction: the credit table and the eager buffers wrap three times
    sends = [np.full(n, (i % 97) + rank, dtype=np.float32) for i, n in enumerate(sizes)]
    recvs = [np.zeros(n, dtype=np.float32) for n in sizes]
    with group():
        for s, r in zip(sends, recvs):
            comm.send(s, peer)
            comm.recv(r, src)
    ok = all(bool((r == (i % 97) + src).all()) for i, r in enumerate(recvs))
    comm.destroy()
    return ok, ctypes.CDLL(os.environ["NCCL_B200_IBV_LIB"]).fake_ib_errors()


def test_many_messages_in_flight_keep_their_order(fake_lib):
    env = dict(BASE, NCCL_NET="IB", NCCL_B200_IBV_LIB=fake_lib, NCCL_B200_IB_EAGER_BYTES="8192")
    res = run_ranks(_many_rank, 2, env=env, timeout=300)
    assert res[0] == (True, 0) and res[1] == (True, 0)


def _peer_leaves(rank, nranks, uid):
    import time
    from nccl_b200 import Communicator, _lib
    comm = Communicator(nranks, rank, uid)
    x = np.ones(1 << 14, dtype=np.float32)
    comm.all_reduce(x)          # one good step over the verbs backend
    if rank == 1:
        os._exit(0)             # leaves between steps: its queue pairs and sockets are gone
    t0 = time.time()
    try:
        comm.all_reduce(x)
        return "ok", 0, time.time() - t0
    except _lib.NcclError as e:
        return "error", e.code, time.time() - t0


def test_peer_that_leaves_turns_into_an_error_over_verbs(fake_lib):
    """The other end's process is gone: the send completes with an error status (the stand-in reports what a real port reports
    after its retries run out), the proxy fails the operation and the collective returns an error instead of waiting forever."""
    env = dict(BASE, NCCL_NET="IB", NCCL_B200_IBV_LIB=fake_lib, NCCL_B200_SOCKET_TIMEOUT_MS="3000")
    res = run_ranks(_peer_leaves, 2, env=env, timeout=90, may_exit=(1,))
    status, code, dt = res[0]
    assert status == "error" and code in (2, 3, 6), res[0]
    assert dt < 30


def _two_node_rank(rank, nranks, uid):
    os.environ["NCCL_HOSTID"] = "node-a" if rank < nranks // 2 else "node-b"   # two ranks per simulated host
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    x = np.full(50000, rank + 1, dtype=np.float32)
    y = np.zeros_like(x)
    comm.all_reduce(x, y)
    g = np.zeros(nranks * 100, dtype=np.float32)
    comm.all_gather(x[:100], g)
    comm.destroy()
    return float(y[0]), float(y[-1]), [float(g[i * 100]) for i in range(nranks)]


def test_ranks_on_two_simulated_hosts_over_verbs(fake_lib, tmp_path):
    """NCCL_HOSTID gives the ranks two host identities: the communicator counts two nodes with two local ranks each, and its
    traffic goes through the verbs backend."""
    env = dict(BASE, NCCL_NET="IB", NCCL_B200_IBV_LIB=fake_lib, NCCL_DEBUG="INFO", NCCL_DEBUG_SUBSYS="INIT,NET", NCCL_DEBUG_FILE=str(tmp_path / "log.%p"))
    res = run_ranks(_two_node_rank, 4, env=env, timeout=300)
    for r in range(4):
        assert res[r] == (10.0, 10.0, [1.0, 2.0, 3.0, 4.0])
    text = "".join(open(tmp_path / f).read() for f in os.listdir(tmp_path))
    assert "nodes 2 localRanks 2" in text and "built-in IB" in text
    # the two ranks of a host take turns over the two devices
    assert text.count("network device 0 of 2") == 2 and text.count("network device 1 of 2") == 2


def _uneven_eager_rank(rank, nranks, uid, sizes):
    os.environ["NCCL_B200_IB_EAGER_BYTES"] = "512" if rank == 0 else "16384"
    return _rank(rank, nranks, uid, sizes)


def test_ends_with_different_eager_sizes_agree_on_the_smaller(fake_lib):
    """A message between the two eager sizes must not be sent eagerly by one end and awaited by credit at the other."""
    env = dict(BASE, NCCL_NET="IB", NCCL_B200_IBV_LIB=fake_lib)
    res = run_ranks(_uneven_eager_rank, 2, args=([100, 500, 2000, 5000],), env=env, timeout=200)
    for r in range(2):
        assert all(res[r][0]) and res[r][1] == 0


def _qps_rank(rank, nranks, uid, sizes, per_rank):
    os.environ["NCCL_IB_QPS_PER_CONNECTION"] = str(per_rank[rank])
    return _rank(rank, nranks, uid, sizes)


@pytest.mark.parametrize("per_rank", [(4, 4, 4), (8, 2, 3)])
def test_messages_split_over_several_queue_pairs(fake_lib, per_rank):
    """RDMA-write messages are cut into one part per queue pair; ends that ask for different numbers use the smaller one.
    Sizes: eager, just above eager (parts of the tail are empty), a size that does not divide evenly, several slices."""
    env = dict(BASE, NCCL_NET="IB", NCCL_B200_IBV_LIB=fake_lib)
    res = run_ranks(_qps_rank, 3, args=([3, 2100, 33333, 1 << 20], per_rank), env=env, timeout=300)
    for r in range(3):
        assert all(res[r][0]) and res[r][1] == 0, res[r]


def test_many_messages_over_several_queue_pairs(fake_lib):
    env = dict(BASE, NCCL_NET="IB", NCCL_B200_IBV_LIB=fake_lib, NCCL_IB_QPS_PER_CONNECTION="3")
    res = run_ranks(_many_rank, 2, env=env, timeout=300)
    assert res[0] == (True, 0) and res[1] == (True, 0)


def test_verbs_requests_are_events_at_the_profiler(fake_lib, tmp_path):
    import json
    plug = os.path.join(ROOT, "nccl_b200", "lib", "plugins", "profiler", "trace.so")
    env = dict(BASE, NCCL_NET="IB", NCCL_B200_IBV_LIB=fake_lib, NCCL_PROFILER_PLUGIN=plug, NCCL_PROFILE_DUMP_FILE=str(tmp_path / "trace"))
    res = run_ranks(_rank, 2, args=([1000, 1 << 16],), env=env, timeout=200)
    assert all(all(res[r][0]) for r in range(2))
    files = [p for p in os.listdir(tmp_path) if p.endswith(".json")]
    ev = json.load(open(os.path.join(tmp_path, files[0])))
    qp = [e for e in ev if e["name"] == "NetIb Qp"]
    assert qp and all(e["cat"] == "NetPlugin" and e["args"]["qp"] > 0 for e in qp)
    # sends by RDMA write with immediate (opcode 1), eager sends (3) and receives (128) all show up
    assert {1, 3, 128} <= {e["args"]["opcode"] for e in qp}


def test_split_and_shrink_build_new_meshes_over_verbs(fake_lib):
    """Every communicator made by split or shrink gets a connection mesh of its own on the verbs backend."""
    import test_api_host
    env = dict(BASE, NCCL_NET="IB", NCCL_B200_IBV_LIB=fake_lib)
    n = 4
    res = run_ranks(test_api_host._splits, n, env=env, timeout=200)
    for r in range(n):
        o = res[r]
        members = [q for q in range(n) if q % 2 == r % 2]
        assert o["sub"][0] == len(members) and o["sub_sum"] == float(sum(members))
        if r != n - 1:
            assert o["shrunk"] == (n - 1, float(n - 1))


def _settings_rank(rank, nranks, uid):
    import ctypes
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    x = np.ones(8, dtype=np.float32)
    comm.all_reduce(x)
    fake = ctypes.CDLL(os.environ["NCCL_B200_IBV_LIB"])
    out = [fake.fake_ib_last(i) for i in range(7)]
    comm.destroy()
    return out


def test_queue_pair_settings_come_from_the_environment(fake_lib):
    env = dict(BASE, NCCL_NET="IB", NCCL_B200_IBV_LIB=fake_lib, NCCL_IB_PKEY="3", NCCL_IB_GID_INDEX="2", NCCL_IB_TC="106", NCCL_IB_SL="5",
               NCCL_IB_TIMEOUT="18", NCCL_IB_RETRY_CNT="4")
    res = run_ranks(_settings_rank, 2, env=env, timeout=120)
    for r in range(2):
        pkey, sgid, tc, sl, timeout, retry, mtu = res[r]
        assert (pkey, sgid, tc, sl, timeout, retry) == (3, 2, 106, 5, 18, 4) and mtu == 5   # 5: 4096-byte path MTU of the stand-in's ports
