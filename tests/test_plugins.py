"""Plugin system on CPU ranks: environment, tuner, profiler (inspector and trace) and network
plugins are loaded from the in-tree example libraries and observed through their side effects."""
import json
import os

import numpy as np
import pytest

from mp_util import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUG = os.path.join(ROOT, "nccl_b200", "lib", "plugins")
BASE = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}


def _rank(rank, nranks, uid, n_iter):
    from nccl_b200 import Communicator, group
    comm = Communicator(nranks, rank, uid)
    x = np.full(1 << 16, rank + 1, dtype=np.float32)
    y = np.zeros_like(x)
    for _ in range(n_iter):
        comm.all_reduce(x, y)
    g = np.zeros(nranks * 128, dtype=np.float32)
    comm.all_gather(x[:128], g)
    peer = (rank + 1) % nranks
    r = np.zeros(256, dtype=np.float32)
    with group():
        comm.send(x[:256], peer)
        comm.recv(r, (rank - 1) % nranks)
    comm.destroy()
    return float(y[0]), float(g[-1]), float(r[0])


def _check(res, n):
    for r in range(n):
        assert res[r][0] == n * (n + 1) / 2
        assert res[r][1] == n
        assert res[r][2] == (r - 1) % n + 1


def test_inspector_plugin_writes_records(tmp_path):
    env = dict(BASE, NCCL_PROFILER_PLUGIN=os.path.join(PLUG, "profiler", "inspector.so"), NCCL_INSPECTOR_DUMP_DIR=str(tmp_path),
               NCCL_INSPECTOR_PROM_DUMP="1", NCCL_INSPECTOR_DUMP_THREAD_INTERVAL_MICROSECONDS="50000")
    _check(run_ranks(_rank, 2, args=(3,), env=env), 2)
    files = sorted(p for p in os.listdir(tmp_path) if p.endswith(".jsonl"))
    assert len(files) == 2
    recs = [json.loads(line) for line in open(os.path.join(tmp_path, files[0]))]
    ar = [r for r in recs if r["func"] == "AllReduce"]
    assert len(ar) == 3 and [r["seq"] for r in ar] == [0, 1, 2]
    assert ar[0]["bytes"] == (1 << 16) * 4 and ar[0]["bus_bw_gbs"] > 0 and ar[0]["nranks"] == 2
    assert any(r["kind"] == "p2p" and r["func"] == "Send" for r in recs)
    prom = [p for p in os.listdir(tmp_path) if p.endswith(".prom")]
    text = open(os.path.join(tmp_path, prom[0])).read()
    assert "nccl_bus_bandwidth_gbs{" in text and 'collective="AllReduce"' in text and "nccl_p2p_count{" in text


def test_trace_plugin_writes_chrome_trace(tmp_path):
    env = dict(BASE, NCCL_PROFILER_PLUGIN=os.path.join(PLUG, "profiler", "trace.so"), NCCL_PROFILE_DUMP_FILE=str(tmp_path / "trace"))
    _check(run_ranks(_rank, 2, args=(1,), env=env), 2)
    files = [p for p in os.listdir(tmp_path) if p.endswith(".json")]
    assert len(files) == 2
    ev = json.load(open(os.path.join(tmp_path, files[0])))
    cats = {e["cat"] for e in ev}
    assert {"CollApi", "Coll", "P2pApi", "P2p", "GroupApi"} <= cats
    assert all(e["dur"] >= 0 for e in ev)


def test_env_plugin_supplies_settings(tmp_path):
    conf = tmp_path / "settings"
    dump = tmp_path / "insp"
    dump.mkdir()
    # the profiler plugin is configured only inside the file: it loads only if the env plugin is consulted
    conf.write_text("NCCL_PROFILER_PLUGIN=%s\n" % os.path.join(PLUG, "profiler", "inspector.so"))
    env = dict(BASE, NCCL_ENV_PLUGIN=os.path.join(PLUG, "env", "file_env.so"), NCCL_ENV_PLUGIN_FILE=str(conf), NCCL_INSPECTOR_DUMP_DIR=str(dump))
    _check(run_ranks(_rank, 2, args=(1,), env=env), 2)
    assert len([p for p in os.listdir(dump) if p.endswith(".jsonl")]) == 2


def test_net_plugin_carries_host_traffic(tmp_path):
    env = dict(BASE, NCCL_NET_PLUGIN=os.path.join(PLUG, "net", "unix_net.so"), NCCL_DEBUG="INFO", NCCL_DEBUG_SUBSYS="NET,INIT",
               NCCL_DEBUG_FILE=str(tmp_path / "log.%p"))
    _check(run_ranks(_rank, 3, args=(2,), env=env), 3)
    logs = "".join(open(os.path.join(tmp_path, p)).read() for p in os.listdir(tmp_path))
    assert "network backend: plugin UnixExample" in logs


def test_builtin_socket_backend_through_proxy():
    env = dict(BASE, NCCL_B200_HOST_NET="1")
    _check(run_ranks(_rank, 3, args=(2,), env=env), 3)


def test_missing_plugin_falls_back(tmp_path):
    env = dict(BASE, NCCL_TUNER_PLUGIN="does-not-exist", NCCL_NET_PLUGIN="none")
    _check(run_ranks(_rank, 2, args=(1,), env=env), 2)


def test_shm_links():
    """Ranks of one host exchange host-memory messages through shared-memory rings."""
    env = dict(BASE, NCCL_B200_HOST_SHM="1", NCCL_B200_HOST_SHM_KB="64")   # small rings: messages wrap many times
    _check(run_ranks(_rank, 3, args=(2,), env=env), 3)


def _collnet_rank(rank, nranks, uid):
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    n = nranks
    x = np.arange(5000, dtype=np.float64) * (rank + 1)
    y = np.zeros_like(x)
    comm.all_reduce(x, y, op="sum")
    z = np.zeros_like(x)
    comm.all_reduce(x, z, op="avg")
    g = np.zeros(n * 300, dtype=np.int32)
    comm.all_gather(np.full(300, rank, dtype=np.int32), g)
    full = np.arange(n * 77, dtype=np.int64) + rank
    part = np.zeros(77, dtype=np.int64)
    comm.reduce_scatter(full, part, op="max")
    half = np.full(64, np.float16(rank + 1), dtype=np.float16)   # a type the fabric does not reduce: falls back to the ring
    hout = np.zeros_like(half)
    comm.all_reduce(half, hout)
    comm.destroy()
    return y, z, g, part, hout


@pytest.mark.parametrize("enable", ["1", "0"])
def test_collective_network_plugin(tmp_path, enable):
    """With NCCL_COLLNET_ENABLE=1 all-reduce / all-gather / reduce-scatter of supported types go through the plugin's
    collective network (its log shows them); unsupported types and NCCL_COLLNET_ENABLE=0 stay on the ring."""
    n = 3
    env = dict(BASE, NCCL_NET_PLUGIN=os.path.join(PLUG, "net", "star_collnet.so"), NCCL_COLLNET_ENABLE=enable,
               STAR_COLLNET_LOG=str(tmp_path / "star"))
    res = run_ranks(_collnet_rank, n, env=env, timeout=200)
    tot = n * (n + 1) / 2
    base = np.arange(5000, dtype=np.float64)
    for r in range(n):
        y, z, g, part, hout = res[r]
        assert np.array_equal(y, base * tot)
        assert np.allclose(z, base * tot / n)
        assert np.array_equal(g, np.repeat(np.arange(n, dtype=np.int32), 300))
        assert np.array_equal(part, np.arange(n * 77, dtype=np.int64)[r * 77:(r + 1) * 77] + n - 1)
        assert np.array_equal(hout, np.full(64, tot, dtype=np.float16))
    logs = [open(os.path.join(tmp_path, p)).read().split() for p in os.listdir(tmp_path)]
    if enable == "1":
        assert len(logs) == n
        for words in logs:
            assert words.count("allreduce") == 2 and words.count("allgather") == 1 and words.count("reducescatter") == 1
    else:
        assert logs == []


def _slow_peer_rank(rank, nranks, uid):
    import os
    import signal
    import time
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    x = np.full(1 << 20, rank + 1, dtype=np.float32)
    if rank == 1:
        time.sleep(1.5)                       # rank 0 sits in its all-reduce meanwhile
    else:
        import threading
        threading.Timer(0.6, lambda: os.kill(os.getpid(), signal.SIGUSR1)).start()
    comm.all_reduce(x)
    comm.destroy()
    return float(x[0])


def test_proxy_state_dump_on_signal(tmp_path):
    """NCCL_PROXY_DUMP_SIGNAL: a signal makes the proxy thread log the operations it has in flight."""
    import signal
    env = dict(BASE, NCCL_B200_HOST_NET="1", NCCL_PROXY_DUMP_SIGNAL=str(int(signal.SIGUSR1)), NCCL_DEBUG="WARN",
               NCCL_DEBUG_FILE=str(tmp_path / "log.%p"))
    res = run_ranks(_slow_peer_rank, 2, env=env, timeout=120)
    assert res[0] == 3.0 and res[1] == 3.0
    logs = "".join(open(os.path.join(tmp_path, p)).read() for p in os.listdir(tmp_path))
    assert "proxy state of rank 0" in logs and "recv from peer 1" in logs


def test_gpu_initiated_networking_table_is_reported(tmp_path):
    """A network plugin library that also exports a table for GPU-initiated networking: the loader initialises it,
    reports what it offers and leaves the traffic where it is."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("needs a C++ compiler")
    so = str(tmp_path / "libunix_gin.so")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-DUNIX_NET_GIN", "-I" + os.path.join(ROOT, "include"),
                           "-I/usr/local/cuda/include", os.path.join(ROOT, "plugins", "net", "unix_net.cc"), "-o", so])
    env = dict(BASE, NCCL_NET_PLUGIN=so, NCCL_DEBUG="INFO", NCCL_DEBUG_SUBSYS="NET,INIT", NCCL_DEBUG_FILE=str(tmp_path / "log.%p"))
    _check(run_ranks(_rank, 2, args=(1,), env=env), 2)
    logs = "".join(open(os.path.join(tmp_path, p)).read() for p in os.listdir(tmp_path) if p.startswith("log."))
    assert "offers GPU-initiated networking UnixExampleGin: 1 device(s), strong signals 1, VA signals 0" in logs
    assert "network backend: plugin UnixExample" in logs


def test_one_library_with_network_and_tuner_plugins(tmp_path):
    """Only NCCL_NET_PLUGIN names the library: the network backend comes from it, and so does the tuner (a tuner that is
    not named by NCCL_TUNER_PLUGIN is looked for in the network plugin's library)."""
    conf = tmp_path / "tuner.conf"
    conf.write_text("allreduce,0,1000000000,ring,simple,2\nallgather,0,4096,ring,ll,-1\n")
    env = dict(BASE, NCCL_NET_PLUGIN=os.path.join(PLUG, "mixed", "mixed_plugin.so"), NCCL_TUNER_CONFIG_FILE=str(conf), NCCL_DEBUG="INFO",
               NCCL_DEBUG_SUBSYS="NET,INIT,TUNING", NCCL_DEBUG_FILE=str(tmp_path / "log.%p"))
    _check(run_ranks(_rank, 2, args=(1,), env=env), 2)
    text = "".join(open(tmp_path / f).read() for f in os.listdir(tmp_path) if f.startswith("log."))
    assert "network backend: plugin" in text and "mixed_plugin.so" in text
    assert "tuner plugin: found in the network plugin's library" in text
    assert "2 rule" in text     # the tuner's own line after reading the configuration file


def test_network_backends_report_their_requests_to_the_profiler(tmp_path):
    """Traffic through the proxy: every slice the socket backend moves is an event of the backend's own kind under the proxy
    operation it belongs to (the backend gets a callback at init and a parent handle with every send / receive)."""
    env = dict(BASE, NCCL_B200_HOST_NET="1", NCCL_PROFILER_PLUGIN=os.path.join(PLUG, "profiler", "trace.so"), NCCL_PROFILE_DUMP_FILE=str(tmp_path / "trace"))
    _check(run_ranks(_rank, 2, args=(1,), env=env), 2)
    files = [p for p in os.listdir(tmp_path) if p.endswith(".json")]
    ev = json.load(open(os.path.join(tmp_path, files[0])))
    net = [e for e in ev if e["cat"] == "NetPlugin"]
    assert net and {e["name"] for e in net} == {"NetSock Send", "NetSock Recv"}
    assert all(e["args"]["bytes"] > 0 and e["args"]["fd"] >= 0 and e["dur"] >= 0 for e in net)
    assert any(e["cat"] == "ProxyOp" for e in ev)
    steps = [e for e in ev if e["cat"] == "ProxyStep"]
    assert steps and all(e["args"]["bytes"] > 0 for e in steps) and len(steps) == len(net)   # one backend request per slice
    ctrl = [e for e in ev if e["cat"] == "ProxyCtrl"]
    assert len(ctrl) == 1 and ctrl[0]["args"]["operations"] == sum(1 for e in ev if e["cat"] == "ProxyOp") and ctrl[0]["args"]["sleeps"] >= 1


@pytest.mark.parametrize("nthreads,nsocks", [(2, 2), (1, 3)])
def test_socket_backend_stripes_messages_over_several_connections(nthreads, nsocks):
    """NCCL_SOCKET_NTHREADS x NCCL_NSOCKS_PERTHREAD connections per comm: large messages are cut over them, small ones stay on the
    first; three ranks dial each other at the same time, so connections of different comms arrive interleaved at a listener."""
    env = dict(BASE, NCCL_B200_HOST_NET="1", NCCL_SOCKET_NTHREADS=str(nthreads), NCCL_NSOCKS_PERTHREAD=str(nsocks))
    res = run_ranks(_stripe_rank, 3, env=env, timeout=200)
    assert all(res[r] for r in range(3))


def _stripe_rank(rank, nranks, uid):
    from nccl_b200 import Communicator, group
    comm = Communicator(nranks, rank, uid)
    ok = True
    for n in (3, 20000, 70001, 1 << 20):      # below the striping threshold, around it, not a multiple of the part size, several slices
        x = (np.arange(n, dtype=np.float32) % 113) + rank
        y = np.zeros_like(x)
        comm.all_reduce(x, y)
        ok = ok and bool(np.array_equal(y, (np.arange(n, dtype=np.float32) % 113) * nranks + nranks * (nranks - 1) / 2))
        s = np.full(n, rank + 1, dtype=np.float32)
        r = np.zeros(n, dtype=np.float32)
        with group():
            comm.send(s, (rank + 1) % nranks)
            comm.recv(r, (rank - 1) % nranks)
        ok = ok and bool((r == (rank - 1) % nranks + 1).all())
    comm.destroy()
    return ok


def test_proxy_threads_run_on_the_named_cpus(tmp_path):
    env = dict(BASE, NCCL_B200_HOST_NET="1", NCCL_PROXY_CPUSET="0", NCCL_SOCKET_RCVBUF="262144", NCCL_SOCKET_SNDBUF="262144", NCCL_DEBUG="INFO",
               NCCL_DEBUG_SUBSYS="INIT,PROXY", NCCL_DEBUG_FILE=str(tmp_path / "log.%p"))
    _check(run_ranks(_rank, 2, args=(1,), env=env), 2)
    text = "".join(open(tmp_path / f).read() for f in os.listdir(tmp_path))
    assert text.count("runs on the CPUs of NCCL_PROXY_CPUSET=0") == 2
