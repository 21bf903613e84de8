#!/usr/bin/env python
"""Headline benchmark: bus bandwidth of a large all-reduce, plus a short sweep of the other collectives.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference]

A step is one ncclAllReduce(sum, bf16) of 1 GiB per rank on registered (symmetric) buffers, the
large-message end of the collective sweep; inputs are synthetic uniform[-1,1] values (seed 7+rank).
N > 1 is launched with one process per GPU (torchrun); rank 0 prints one JSON line.

  value       nccl-tests bus bandwidth, GB/s: bytes/time * 2(n-1)/n. With one GPU that factor is
              zero, so the n=1 line reports the algorithm bandwidth of the one-rank path instead.
  e2e         the same step from and to pinned host memory: every step copies the 1 GiB input host->device,
              all-reduces it and copies the result device->host. Our arm makes the library's call for that
              (Communicator.all_reduce_from_host = ncclAllReduceFromHost: the three stages overlap chunk by
              chunk); the reference arm issues the three operations one after the other on one stream, which
              is what its API offers.
  sweep       time and bus bandwidth of all-reduce / all-gather / reduce-scatter / all-to-all /
              broadcast / send-recv at a few sizes, bf16 and fp32 (20 warm-up + 100 timed calls per
              point up to 64 MiB, fewer above; the faster of two timed passes).
  verified    outside the timed regions the headline result and every sweep point are compared on the
              device with an fp32 PyTorch computation over inputs regenerated from the seeds of all
              ranks; a mismatch makes the run exit non-zero.
  --full      the whole configured sweep: 8 B to 8 GiB doubling, both dtypes (slow; not the default).

--impl reference runs the same driver against the library built from the reference sources
(baseline/_ref/build/lib/libnccl.so.2) through its public C API.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
REF_LIB = os.path.join(ROOT, "baseline", "_ref", "build", "lib", "libnccl.so.2")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--bytes", type=int, default=1 << 30)
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--full", action="store_true", help="sweep every size from 8 B to --full-max (default 8 GiB), doubling, bf16 and fp32")
    ap.add_argument("--full-max", type=int, default=8 << 30)
    ap.add_argument("--full-out", default=None, help="also write the full sweep to this file")
    ap.add_argument("--env", action="append", default=[], help="KEY=VALUE set before the library is loaded (e.g. NCCL_SYM_TMA_ENABLE=1 for the reference)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    for kv in a.env:
        k, _, v = kv.partition("=")
        os.environ[k] = v

    if a.impl == "reference" and not os.path.exists(REF_LIB):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/build/lib/libnccl.so.2 is missing (reference was not built in this checkout)"}))
        return 0

    import torch
    from nccl_b200 import _lib
    from nccl_b200.core import BF16, FP32
    from nccl_b200.utils import perf

    d = perf.Dist()
    n = d.world
    if n != a.gpus and d.rank == 0:
        print("warning: --gpus %d but WORLD_SIZE %d" % (a.gpus, n), file=sys.stderr)
    torch.cuda.set_device(d.local_rank)
    lib = _lib.load(REF_LIB) if a.impl == "reference" else _lib.load()
    nbytes = a.bytes
    h = perf.Harness(d, lib, max_bytes=max(nbytes, a.full_max if a.full else 0), symmetric=True)
    h.fill(BF16)

    # ---------------- device-timed headline: K all-reduces back to back
    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else
                           os.environ["CUDA_VISIBLE_DEVICES"].split(",")[torch.cuda.current_device()])
    launches0 = 0
    count_launches = a.impl == "ours" and hasattr(lib, "b200CommLaunchCount")
    if count_launches:
        lib.b200CommLaunchCount.restype = ctypes.c_ulonglong
        lib.b200CommLaunchCount.argtypes = [ctypes.c_void_p]
    sp = h.stream.cuda_stream
    with torch.cuda.stream(h.stream):
        for _ in range(a.warmup):
            _lib.check(h.call("all_reduce", nbytes, BF16, sp), "ncclAllReduce", lib)
    d.barrier()
    torch.cuda.synchronize()
    if count_launches:
        launches0 = lib.b200CommLaunchCount(h.comm)
    if d.rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(h.stream):
        e0.record(h.stream)
        for _ in range(a.steps):
            _lib.check(h.call("all_reduce", nbytes, BF16, sp), "ncclAllReduce", lib)
        e1.record(h.stream)
    torch.cuda.synchronize()
    d.barrier()
    clocks = sampler.stop() if d.rank == 0 else None
    ms = d.max(e0.elapsed_time(e1) / a.steps)
    launches = (lib.b200CommLaunchCount(h.comm) - launches0) if count_launches else None
    factor = perf.bus_factor("all_reduce", n)
    value = nbytes / (ms * 1e-3) / 1e9 * factor

    # ---------------- the headline result, checked against the seeds of all ranks (not timed)
    ver = perf.Verifier(h, BF16, 256 << 20)
    ver.check("all_reduce", nbytes)

    # ---------------- end to end: pinned host -> device, all-reduce through the public API, device -> host
    e2e = None
    try:
        host_in = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
        host_out = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
        host_in.view(torch.bfloat16).copy_(h.send_t.view(torch.bfloat16).cpu())
        if a.impl == "ours":
            from nccl_b200.core import Communicator
            api = Communicator(n, d.rank, None, lib=lib, _handle=h.comm)
            send_bf, recv_bf = h.send_t.view(torch.bfloat16), h.recv_t.view(torch.bfloat16)

            hin_bf, hout_bf = host_in.view(torch.bfloat16), host_out.view(torch.bfloat16)

            def step():
                # the library's call for host-resident data: copy in, all-reduce and copy out, overlapped chunk by chunk
                api.all_reduce_from_host(hin_bf, hout_bf, send_bf, recv_bf, op="sum", stream=h.stream)
        else:
            def step():
                h.send_t.copy_(host_in, non_blocking=True)
                _lib.check(h.call("all_reduce", nbytes, BF16, sp), "ncclAllReduce", lib)
                host_out.copy_(h.recv_t, non_blocking=True)
        k2 = max(3, min(a.steps, 10))
        with torch.cuda.stream(h.stream):
            for _ in range(3):
                step()
        torch.cuda.synchronize()
        d.barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(h.stream):
            f0.record(h.stream)
            for _ in range(k2):
                step()
            f1.record(h.stream)
        torch.cuda.synchronize()
        ms2 = d.max(f0.elapsed_time(f1) / k2)
        # what arrived in host memory is what the device holds (head and tail of the buffer), and the device result is
        # checked against the seeds like the headline above
        span = min(nbytes, 64 << 20)
        same = bool(torch.equal(host_out[:span].cuda(), h.recv_t[:span])) and bool(torch.equal(host_out[nbytes - span:].cuda(), h.recv_t[nbytes - span:nbytes]))
        ver.check("all_reduce", nbytes)
        e2e = {"value": round(nbytes / (ms2 * 1e-3) / 1e9 * factor, 3), "unit": "GB/s", "ms_per_step": round(ms2, 4), "steps": k2,
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "host_result_matches_device": same}
        if not same:
            ver.failures.append("e2e: host result differs from the device result")
    except Exception as ex:  # noqa: BLE001
        e2e = {"error": str(ex)[:200]}

    # ---------------- short sweep (time and bus bandwidth at a few sizes, registered buffers), every point verified
    sweep = sweep32 = full = None
    colls = ("all_reduce", "all_gather", "reduce_scatter", "all_to_all", "broadcast", "sendrecv")

    def run_sweep(dt, verifier, sizes, iters):
        res = {}
        for coll in colls:
            try:
                rows = perf.sweep(h, coll, dt, sizes, warmup=20, iters=iters, verifier=verifier)
                res[coll] = {str(r["bytes"]): [r["time_us"], r["busbw_GBps"]] for r in rows}
            except Exception as ex:  # noqa: BLE001
                res[coll] = {"error": str(ex)[:200]}
        return res

    ver32 = None
    if not a.no_sweep and n > 1:
        sizes = [s for s in (8, 1 << 10, 32 << 10, 1 << 20, 16 << 20, 256 << 20) if s <= nbytes]
        sweep = run_sweep(BF16, ver, sizes, 100)
        if a.full:
            full = {"bf16": run_sweep(BF16, ver, [1 << k for k in range(3, 40) if (1 << k) <= a.full_max], 100)}
        h.fill(FP32)
        ver32 = perf.Verifier(h, FP32, 256 << 20)
        sweep32 = run_sweep(FP32, ver32, [s for s in (8, 32 << 10, 1 << 20, 64 << 20) if s <= nbytes], 100)
        if a.full:
            full["fp32"] = run_sweep(FP32, ver32, [1 << k for k in range(3, 40) if (1 << k) <= a.full_max], 100)
    verified = ver.summary()
    if ver32 is not None:
        v32 = ver32.summary()
        verified = {"ok": verified["ok"] and v32["ok"], "points": verified["points"] + v32["points"],
                    "max_abs_err": {"bf16": verified["max_abs_err"], "fp32": v32["max_abs_err"]}, "failures": (verified["failures"] + v32["failures"])[:4]}
    ver = ver32 = None
    h.close()
    if d.rank == 0:
        out = {
            "metric": "allreduce_busbw_GBps", "value": round(value, 3), "unit": "GB/s", "n_gpus": n, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform[-1,1], seed 7+rank", "impl": a.impl,
            "config": {"model": "collective sweep, large-message point", "collective": "AllReduce", "op": "sum",
                       "bytes_per_rank": nbytes, "global_batch": n, "seq_len": nbytes // 2, "parallelism": "dp%d" % n,
                       "buffers": "ncclMemAlloc + ncclCommWindowRegister(NCCL_WIN_COLL_SYMMETRIC)",
                       "l2": "1 GiB per rank per step: inputs larger than the 126 MB L2, no flush needed",
                       "busbw": "algBW*2(n-1)/n" if n > 1 else "n=1: algBW of the one-rank copy path (the bus factor is 0)",
                       "sweep_call_loop": "C loop over the library's entry points (tools/perf_loop.c), the same for both arms" if h._native_loop() is not None
                       else "interpreter loop (ctypes call per collective)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "verified": verified, "sweep_time_us_busbw": sweep,
            "sweep_fp32_time_us_busbw": sweep32,
        }
        if full is not None:
            out["full_sweep_time_us_busbw"] = full
            if a.full_out:
                with open(a.full_out, "w") as f:
                    json.dump({"impl": a.impl, "n_gpus": n, "env": a.env, "full": full, "verified": verified}, f)
        print(json.dumps(out))
    if not verified["ok"]:
        if d.rank == 0:
            print("bench.py: results do not match the values recomputed from the seeds: %s" % verified["failures"], file=sys.stderr)
        return 3
    return 0


if __name__ == "__main__":
    sys.exit(main())
