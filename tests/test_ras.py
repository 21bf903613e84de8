"""RAS thread: status reports through the client socket, operation-count mismatch detection, and
dead-process detection after a rank's process has gone away (host-side failure, no GPU)."""
import json
import os
import socket
import subprocess
import time

import numpy as np

from mp_util import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NCCLRAS = os.path.join(ROOT, "nccl_b200", "bin", "ncclras")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _query(port, fmt="json", verbose=False):
    cmd = [NCCLRAS, "-h", "127.0.0.1", "-p", str(port), "-t", "2", "-f", fmt] + (["-v"] if verbose else [])
    return subprocess.run(cmd, capture_output=True, text=True, timeout=60).stdout


def _status_rank(rank, nranks, uid, port):
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    x = np.ones(1024, dtype=np.float32)
    for _ in range(3):
        comm.all_reduce(x.copy(), x)
    out = None
    if rank == 0:
        time.sleep(0.3)
        out = (_query(port, "json"), _query(port, "text", verbose=True))
    # everyone stays until rank 0 has its report
    comm.all_reduce(np.ones(4, dtype=np.float32))
    comm.destroy()
    return out


def test_status_report():
    port = _free_port()
    env = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo", "NCCL_RAS_ADDR": "127.0.0.1:%d" % port}
    res = run_ranks(_status_rank, 3, args=(port,), env=env)
    js, text = res[0]
    rep = json.loads(js)
    assert rep["job"]["processes"] == 3 and rep["job"]["dead_processes"] == 0
    assert len(rep["communicators"]) == 1
    c = rep["communicators"][0]
    assert c["nranks"] == 3 and c["status"] == "RUNNING" and c["missing_ranks"] == 0 and c["op_count"] >= 3
    assert "Job summary" in text and "Communicators" in text and "rank 2: pid" in text


def _dead_rank(rank, nranks, uid, port, done_file):
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    comm.all_reduce(np.ones(16, dtype=np.float32))
    if rank == 2:
        os._exit(0)     # leaves between steps, nothing in flight; its RAS thread dies with it
    out = None
    if rank == 0:
        deadline = time.time() + 30
        while time.time() < deadline:
            raw = _query(port, "json")
            if not raw:      # the process that served the client port has just gone; another one takes it over
                time.sleep(0.3)
                continue
            try:
                rep = json.loads(raw)
            except ValueError:   # the serving process went away in the middle of a reply
                time.sleep(0.3)
                continue
            if rep["job"]["dead_processes"] >= 1:
                out = rep
                break
            time.sleep(0.3)
        open(done_file, "w").close()
    else:
        deadline = time.time() + 40
        while not os.path.exists(done_file) and time.time() < deadline:   # stay alive until rank 0 has its report
            time.sleep(0.1)
    return out


def test_dead_process_is_reported(tmp_path):
    port = _free_port()
    env = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo", "NCCL_RAS_ADDR": "127.0.0.1:%d" % port,
           "NCCL_B200_RAS_KEEPALIVE_MS": "100", "NCCL_B200_RAS_DEAD_AFTER": "3"}
    res = run_ranks(_dead_rank, 3, args=(port, str(tmp_path / "done")), env=env, timeout=120, may_exit=(2,))
    rep = res[0]
    assert rep is not None, "the dead process was never reported"
    assert rep["job"]["dead_processes"] == 1 and rep["job"]["processes"] == 2
    assert rep["communicators"][0]["status"] == "INCOMPLETE" and rep["communicators"][0]["missing_ranks"] == 1
    assert any("DEAD" in e for e in rep["errors"])


def _monitor_rank(rank, nranks, uid, port):
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    comm.all_reduce(np.ones(4, dtype=np.float32))
    mon = None
    if rank == 0:
        mon = subprocess.Popen([NCCLRAS, "--host", "127.0.0.1", "--port", str(port), "--monitor=lifecycle"], stdout=subprocess.PIPE, text=True)
        time.sleep(0.6)
    comm.all_reduce(np.ones(4, dtype=np.float32))   # the monitor is connected before anything happens
    sub = comm.split(0, rank)                        # every process creates and destroys a communicator
    sub.all_reduce(np.ones(4, dtype=np.float32))
    sub.destroy()
    comm.all_reduce(np.ones(4, dtype=np.float32))
    out = None
    if rank == 0:
        time.sleep(0.8)
        mon.terminate()
        out = mon.communicate(timeout=10)[0]
    comm.all_reduce(np.ones(4, dtype=np.float32))
    comm.destroy()
    return out


def test_monitor_mode_streams_events():
    """ncclras --monitor keeps its connection and prints one line per event of the serving process."""
    port = _free_port()
    env = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo", "NCCL_RAS_ADDR": "127.0.0.1:%d" % port}
    res = run_ranks(_monitor_rank, 2, args=(port,), env=env, timeout=120)
    lines = [l for l in res[0].splitlines() if l.strip()]
    assert any(" lifecycle communicator " in l and l.endswith("created") for l in lines), lines
    assert any(" lifecycle communicator " in l and l.endswith("destroyed") for l in lines), lines
    assert all(float(l.split()[0]) > 1e9 for l in lines)   # every event carries its wall-clock time


def test_client_options():
    assert "--monitor" in subprocess.run([NCCLRAS, "--help"], capture_output=True, text=True).stdout
    assert subprocess.run([NCCLRAS, "--version"], capture_output=True, text=True).stdout.startswith("ncclras ")
    assert subprocess.run([NCCLRAS, "--no-such-option"], capture_output=True, text=True).returncode == 2
