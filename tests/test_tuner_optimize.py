"""The script that turns measurements into a configuration for the CSV tuner plugin, and the plugin reading its output."""
import os
import subprocess
import sys

from mp_util import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "plugins", "tuner", "optimize_config.py")

DATA = """collective,size_bytes,algorithm,protocol,channels,nodes,ranks,pipeOps,regBuff,cost_metric,bandwidth_gbps,latency_us
# two choices per size; latency and bandwidth disagree at 65536
allreduce,1024,tree,ll,2,1,2,-1,-1,0.2,1.0,6.0
allreduce,1024,ring,simple,4,1,2,-1,-1,0.3,0.8,9.0
allreduce,4096,tree,ll,2,1,2,-1,-1,0.2,3.0,7.0
allreduce,4096,ring,simple,4,1,2,-1,-1,0.4,2.0,10.0
allreduce,65536,tree,ll,2,1,2,-1,-1,0.5,20.0,14.0
allreduce,65536,ring,simple,4,1,2,-1,-1,0.6,25.0,15.0
allreduce,1048576,tree,ll,2,1,2,-1,-1,0.9,60.0,40.0
allreduce,1048576,ring,simple,4,1,2,-1,-1,0.7,90.0,30.0
broadcast,1024,ring,simple,1,2,16,-1,-1,0.1,1.0,5.0
"""


def _run(tmp_path, *args):
    src = tmp_path / "perf.csv"
    src.write_text(DATA)
    p = subprocess.run([sys.executable, SCRIPT, str(src), *args], capture_output=True, text=True, timeout=60)
    assert p.returncode == 0, p.stderr
    return p.stdout


def test_runs_of_one_choice_are_merged_and_borders_sit_between_sizes(tmp_path):
    out = _run(tmp_path, "--dry-run", "-m", "latency_us", "--no-header").strip().splitlines()
    # tree/ll wins up to 65536, ring/simple at 1 MiB: the border is the geometric mean of 65536 and 1048576 = 262144
    assert out == ["allreduce,0,262144,tree,ll,2,1,2,-1,-1", "allreduce,262145,%d,ring,simple,4,1,2,-1,-1" % (1 << 62), "broadcast,0,%d,ring,simple,1,2,16,-1,-1" % (1 << 62)]
    bw = _run(tmp_path, "--dry-run", "-m", "bandwidth_gbps", "--no-header").strip().splitlines()
    # by bandwidth ring/simple already wins at 65536: border between 4096 and 65536 = 16384
    assert bw[0] == "allreduce,0,16384,tree,ll,2,1,2,-1,-1" and bw[1].startswith("allreduce,16385,")


def test_missing_columns_are_reported(tmp_path):
    bad = tmp_path / "bad.csv"
    bad.write_text("collective,size_bytes\nallreduce,8\n")
    p = subprocess.run([sys.executable, SCRIPT, str(bad)], capture_output=True, text=True, timeout=60)
    assert p.returncode != 0 and "missing column" in p.stderr


def _rank(rank, nranks, uid):
    import numpy as np
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    x = np.ones(64, dtype=np.float32)
    y = np.zeros_like(x)
    comm.all_reduce(x, y)
    comm.destroy()
    return float(y[0])


def test_the_plugin_reads_what_the_script_writes(tmp_path):
    conf = tmp_path / "nccl_tuner.conf"
    out = _run(tmp_path, "-o", str(conf))
    assert "3 rule(s) written" in out
    env = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo", "NCCL_TUNER_PLUGIN": os.path.join(ROOT, "nccl_b200", "lib", "plugins", "tuner", "csv_tuner.so"),
           "NCCL_TUNER_CONFIG_FILE": str(conf), "NCCL_DEBUG": "INFO", "NCCL_DEBUG_SUBSYS": "TUNING,INIT", "NCCL_DEBUG_FILE": str(tmp_path / "log.%p")}
    res = run_ranks(_rank, 2, env=env)
    assert res[0] == res[1] == 2.0
    text = "".join(open(tmp_path / f).read() for f in os.listdir(tmp_path) if f.startswith("log."))
    assert "csv tuner: 3 rule(s)" in text
