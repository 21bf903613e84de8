"""Tuner and profiler plugins on GPU communicators: the CSV tuner steers the algorithm choice and
the inspector reports it together with device-side timings."""
import json
import os

import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUG = os.path.join(ROOT, "nccl_b200", "lib", "plugins")


def _rank(rank, nranks, uid):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    x = torch.full((1 << 20,), float(rank + 1), device="cuda")
    y = torch.zeros_like(x)
    for _ in range(3):
        comm.all_reduce(x, y)
    torch.cuda.synchronize()
    small = torch.ones(64, device="cuda")
    comm.all_reduce(small)
    torch.cuda.synchronize()
    out = (float(y[0]), float(small[0]))
    comm.destroy()
    return out


@pytest.mark.parametrize("n", [1, 2])
def test_tuner_and_inspector(n, tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    conf = tmp_path / "tuner.conf"
    conf.write_text("# collective,min,max,algo,proto,channels\nallreduce,1024,1000000000,ring,simple,4\n")
    env = {"NCCL_TUNER_PLUGIN": os.path.join(PLUG, "tuner", "csv_tuner.so"), "NCCL_TUNER_CONFIG_FILE": str(conf),
           "NCCL_PROFILER_PLUGIN": os.path.join(PLUG, "profiler", "inspector.so"), "NCCL_INSPECTOR_DUMP_DIR": str(tmp_path)}
    res = run_ranks(_rank, n, env=env)
    for r in range(n):
        assert res[r] == (n * (n + 1) / 2, float(n))
    files = sorted(p for p in os.listdir(tmp_path) if p.endswith(".jsonl"))
    assert len(files) == n
    recs = [json.loads(line) for line in open(os.path.join(tmp_path, files[0]))]
    big = [r for r in recs if r["func"] == "AllReduce" and r["count"] == 1 << 20]
    assert len(big) == 3
    assert all(r["timing"] == "device" and r["exec_time_us"] > 0 for r in big)
    if n > 1:
        assert all(r["algo"] == "RING" and r["channels"] == 4 for r in big), big
        small = [r for r in recs if r["count"] == 64]
        assert small and small[0]["algo"] != "RING"   # below the rule's size range: built-in choice


def test_kernel_events_carry_device_time_stamps(tmp_path):
    """Every CTA of a collective kernel stamps its start and stop with the GPU's global timer; the profiler
    glue turns them into one KernelCh event per CTA under the collective's event."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = {"NCCL_PROFILER_PLUGIN": os.path.join(PLUG, "profiler", "trace.so"), "NCCL_PROFILE_DUMP_FILE": str(tmp_path / "trace")}
    res = run_ranks(_rank, 2, env=env)
    assert res[0] == (3.0, 2.0)
    files = sorted(p for p in os.listdir(tmp_path) if p.endswith(".json"))
    assert len(files) == 2
    for f in files:
        ev = json.load(open(os.path.join(tmp_path, f)))
        colls = [e for e in ev if e["cat"] == "Coll"]
        chans = [e for e in ev if e["cat"] == "KernelCh"]
        assert len(colls) == 4 and len(chans) >= 4
        ids = set()
        for e in chans:
            a = e["args"]
            ids.add(a["channel"])
            assert 0 < a["gpu_start_ns"] <= a["gpu_stop_ns"] < a["gpu_start_ns"] + 200_000_000, a
        assert len(ids) > 1, "the 4 MiB all-reduce runs on several CTAs, each with its own record"
        # the three large calls ran one after the other on the stream: their device windows do not overlap
        spans = sorted((e["args"]["gpu_start_ns"], e["args"]["gpu_stop_ns"]) for e in chans if e["args"]["channel"] == 0)
        assert all(spans[i][1] <= spans[i + 1][0] + 50_000 for i in range(len(spans) - 1)), spans
