"""Collective performance harness with the nccl-tests conventions.

Runs one collective through the NCCL C API of a chosen library (this package's or any other
libnccl.so with the same ABI), times it on the device with CUDA events, takes the maximum over
ranks, and reports algorithm and bus bandwidth:

    algBW = bytes / time
    busBW = algBW * 2(n-1)/n   all-reduce
          = algBW * (n-1)/n    all-gather, reduce-scatter, all-to-all
          = algBW              broadcast, reduce, send/recv

Launched one process per GPU (torchrun); torch.distributed (gloo) carries the unique id and the
max-over-ranks of the timings. Can be run as a module:  torchrun ... -m nccl_b200.utils.perf --coll all_reduce
"""
import argparse
import ctypes
import json
import os
import sys

import torch

from .. import _lib
from ..core import BF16, FP32, TYPE_SIZE

COLLS = ("all_reduce", "all_gather", "reduce_scatter", "broadcast", "all_to_all", "reduce", "sendrecv")


class _Raw:
    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def tensor_at(ptr, nbytes):
    """uint8 CUDA tensor aliasing device memory at `ptr` (no copy, no ownership)."""
    return torch.as_tensor(_Raw(ptr, nbytes), device="cuda")


def bus_factor(coll, n):
    if n == 1:
        return 1.0  # a single rank only copies: report the algorithm bandwidth
    if coll == "all_reduce":
        return 2.0 * (n - 1) / n
    if coll in ("all_gather", "reduce_scatter", "all_to_all"):
        return (n - 1) / n
    return 1.0


class Dist:
    """torch.distributed plumbing (gloo): unique-id broadcast and max-reduction of timings."""

    def __init__(self):
        import torch.distributed as dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = dist
        if self.world > 1 and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
            dist.init_process_group(backend="gloo", rank=self.rank, world_size=self.world)

    def bcast_bytes(self, raw):
        if self.world == 1:
            return raw
        obj = [raw]
        self.dist.broadcast_object_list(obj, src=0)
        return obj[0]

    def max(self, value):
        if self.world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t[0])

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()


class Harness:
    """A communicator of `lib` plus buffers, for timing collectives at many sizes."""

    def __init__(self, dist, lib=None, max_bytes=1 << 30, symmetric=True):
        self.d = dist
        self.lib = lib or _lib.load()
        self.n = dist.world
        self.rank = dist.rank
        torch.cuda.set_device(dist.local_rank)
        self.stream = torch.cuda.Stream()
        uid = _lib.ncclUniqueId()
        if dist.rank == 0:
            _lib.check(self.lib.ncclGetUniqueId(ctypes.byref(uid)), "ncclGetUniqueId", self.lib)
        raw = dist.bcast_bytes(ctypes.string_at(ctypes.byref(uid), 128))
        ctypes.memmove(ctypes.byref(uid), raw, 128)
        self.comm = _lib.ncclComm_t()
        _lib.check(self.lib.ncclCommInitRank(ctypes.byref(self.comm), self.n, uid, self.rank), "ncclCommInitRank", self.lib)
        self.symmetric = symmetric
        self.max_bytes = max_bytes
        self.send_bytes = max_bytes
        self.recv_bytes = max_bytes
        self.wins = []
        if symmetric:
            self.send_ptr = self._alloc(self.send_bytes)
            self.recv_ptr = self._alloc(self.recv_bytes)
            for p, b in ((self.send_ptr, self.send_bytes), (self.recv_ptr, self.recv_bytes)):
                w = ctypes.c_void_p()
                _lib.check(self.lib.ncclCommWindowRegister(self.comm, p, b, ctypes.byref(w), 1), "ncclCommWindowRegister", self.lib)
                self.wins.append(w)
            self.send_t = tensor_at(self.send_ptr, self.send_bytes)
            self.recv_t = tensor_at(self.recv_ptr, self.recv_bytes)
        else:
            self.send_t = torch.empty(self.send_bytes, dtype=torch.uint8, device="cuda")
            self.recv_t = torch.empty(self.recv_bytes, dtype=torch.uint8, device="cuda")
            self.send_ptr, self.recv_ptr = self.send_t.data_ptr(), self.recv_t.data_ptr()

    def _alloc(self, nbytes):
        p = ctypes.c_void_p()
        _lib.check(self.lib.ncclMemAlloc(ctypes.byref(p), nbytes), "ncclMemAlloc", self.lib)
        return p.value

    def fill(self, dtype_code, seed=7):
        """uniform[-1, 1] with seed 7 + rank, as the sweep configuration prescribes."""
        g = torch.Generator(device="cuda").manual_seed(seed + self.rank)
        tdt = torch.bfloat16 if dtype_code == BF16 else torch.float32
        view = self.send_t.view(tdt)
        step = 1 << 26
        for i in range(0, view.numel(), step):
            chunk = view[i:i + step]
            chunk.copy_((torch.rand(chunk.numel(), generator=g, device="cuda", dtype=torch.float32) * 2 - 1).to(tdt))

    def call(self, coll, nbytes, dtype_code, stream_ptr):
        """Issues one collective whose per-rank message is `nbytes` (nccl-tests size convention)."""
        es = TYPE_SIZE[dtype_code]
        L, c, n = self.lib, self.comm, self.n
        if coll == "all_reduce":
            return L.ncclAllReduce(self.send_ptr, self.recv_ptr, nbytes // es, dtype_code, 0, c, stream_ptr)
        if coll == "all_gather":   # nbytes = total received
            return L.ncclAllGather(self.send_ptr, self.recv_ptr, nbytes // es // n, dtype_code, c, stream_ptr)
        if coll == "reduce_scatter":   # nbytes = total sent
            return L.ncclReduceScatter(self.send_ptr, self.recv_ptr, nbytes // es // n, dtype_code, 0, c, stream_ptr)
        if coll == "all_to_all":
            return L.ncclAlltoAll(self.send_ptr, self.recv_ptr, nbytes // es // n, dtype_code, c, stream_ptr)
        if coll == "broadcast":
            return L.ncclBroadcast(self.send_ptr, self.recv_ptr, nbytes // es, dtype_code, 0, c, stream_ptr)
        if coll == "reduce":
            return L.ncclReduce(self.send_ptr, self.recv_ptr, nbytes // es, dtype_code, 0, 0, c, stream_ptr)
        if coll == "sendrecv":
            nxt, prv = (self.rank + 1) % n, (self.rank - 1) % n
            L.ncclGroupStart()
            L.ncclSend(self.send_ptr, nbytes // es, dtype_code, nxt, c, stream_ptr)
            L.ncclRecv(self.recv_ptr, nbytes // es, dtype_code, prv, c, stream_ptr)
            return L.ncclGroupEnd()
        raise ValueError(coll)

    def time(self, coll, nbytes, dtype_code=FP32, warmup=20, iters=100, min_warm_ms=3.0):
        """Mean device time per call in microseconds (max over ranks). The warm-up covers at least
        `warmup` calls and roughly `min_warm_ms` of device time: after the host-side barrier between
        two measurements the GPU has been idle and its clocks have dropped, and a window of a few
        short kernels would otherwise be timed at idle clocks. The number of warm-up calls is a
        function of the message size only, so every rank issues the same sequence of collectives."""
        sp = self.stream.cuda_stream
        est_us = 10.0 + nbytes / 3.0e5                       # rough per-call time: 10 us + bytes at 300 GB/s
        warm = max(warmup, min(2000, int(min_warm_ms * 1e3 / est_us) + 1))
        with torch.cuda.stream(self.stream):
            self.d.barrier()
            for _ in range(warm):
                _lib.check(self.call(coll, nbytes, dtype_code, sp), coll, self.lib)
            self.stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(iters):
                _lib.check(self.call(coll, nbytes, dtype_code, sp), coll, self.lib)
            e1.record(self.stream)
            self.stream.synchronize()
        us = e0.elapsed_time(e1) * 1000.0 / iters
        return self.d.max(us)

    def time_host(self, coll, nbytes, dtype_code=FP32, iters=200):
        """Host time per call in microseconds (max over ranks): how long the calling thread spends
        inside the library per collective while the device queue is not full."""
        import time as _time
        sp = self.stream.cuda_stream
        with torch.cuda.stream(self.stream):
            self.d.barrier()
            for _ in range(20):
                _lib.check(self.call(coll, nbytes, dtype_code, sp), coll, self.lib)
            self.stream.synchronize()
            t0 = _time.perf_counter()
            for _ in range(iters):
                self.call(coll, nbytes, dtype_code, sp)
            t1 = _time.perf_counter()
            self.stream.synchronize()
        return self.d.max((t1 - t0) * 1e6 / iters)

    def time_graph(self, coll, nbytes, dtype_code=FP32, calls=50, replays=5):
        """Mean device time per call when `calls` collectives are captured into one CUDA graph and
        the graph is replayed: launch cost on the host no longer limits the rate."""
        sp = self.stream.cuda_stream
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self.stream):
            self.d.barrier()
            for _ in range(5):
                _lib.check(self.call(coll, nbytes, dtype_code, sp), coll, self.lib)
            self.stream.synchronize()
        with torch.cuda.graph(g, stream=self.stream):
            for _ in range(calls):
                _lib.check(self.call(coll, nbytes, dtype_code, self.stream.cuda_stream), coll, self.lib)
        with torch.cuda.stream(self.stream):
            self.d.barrier()
            g.replay()
            self.stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(replays):
                g.replay()
            e1.record(self.stream)
            self.stream.synchronize()
        us = e0.elapsed_time(e1) * 1000.0 / (replays * calls)
        return self.d.max(us)

    def close(self):
        torch.cuda.synchronize()
        for w in self.wins:
            self.lib.ncclCommWindowDeregister(self.comm, w)
        if self.symmetric:
            self.send_t = self.recv_t = None
            self.lib.ncclMemFree(ctypes.c_void_p(self.send_ptr))
            self.lib.ncclMemFree(ctypes.c_void_p(self.recv_ptr))
        self.lib.ncclCommDestroy(self.comm)


def sweep(h, coll, dtype_code, sizes, warmup=20, iters=100):
    rows = []
    for nbytes in sizes:
        es = TYPE_SIZE[dtype_code]
        unit = es * (h.n if coll in ("all_gather", "reduce_scatter", "all_to_all") else 1)
        nb = max(unit, nbytes // unit * unit)
        if nb > h.max_bytes:
            break
        it = iters if nb <= (64 << 20) else max(5, iters // 10)
        wu = warmup if nb <= (64 << 20) else max(3, warmup // 5)
        us = h.time(coll, nb, dtype_code, wu, it)
        alg = nb / us / 1e3
        rows.append({"bytes": nb, "time_us": round(us, 2), "algbw_GBps": round(alg, 2), "busbw_GBps": round(alg * bus_factor(coll, h.n), 2)})
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--coll", default="all_reduce", choices=COLLS)
    ap.add_argument("--dtype", default="fp32", choices=("fp32", "bf16"))
    # (--min / --max also work when the module is not started through torchrun, whose own parser claims "--max")
    ap.add_argument("--minbytes", "--min", dest="min", type=int, default=8)
    ap.add_argument("--maxbytes", "--max", dest="max", type=int, default=1 << 30)
    ap.add_argument("--lib", default=None, help="path of another libnccl.so to measure instead of this package's library")
    ap.add_argument("--plain", action="store_true", help="cudaMalloc buffers instead of registered symmetric windows")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--out", default=None)
    ap.add_argument("--latency", action="store_true", help="per size: host time per call, device time per call issued eagerly, and replayed from a CUDA graph")
    a = ap.parse_args(argv)
    d = Dist()
    lib = _lib.load(a.lib) if a.lib else _lib.load()
    h = Harness(d, lib, max_bytes=a.max, symmetric=not a.plain)
    dt = BF16 if a.dtype == "bf16" else FP32
    h.fill(dt)
    sizes = []
    s = a.min
    while s <= a.max:
        sizes.append(s)
        s *= 2
    if a.latency:
        rows = []
        es = TYPE_SIZE[dt]
        unit = es * (h.n if a.coll in ("all_gather", "reduce_scatter", "all_to_all") else 1)
        for nbytes in sizes:
            nb = max(unit, nbytes // unit * unit)
            row = {"bytes": nb, "eager_us": round(h.time(a.coll, nb, dt, a.warmup, a.iters), 2), "host_us": round(h.time_host(a.coll, nb, dt), 2)}
            try:
                row["graph_us"] = round(h.time_graph(a.coll, nb, dt), 2)
            except Exception as ex:  # noqa: BLE001
                row["graph_error"] = str(ex)[:120]
            rows.append(row)
    else:
        rows = sweep(h, a.coll, dt, sizes, a.warmup, a.iters)
    h.close()
    if d.rank == 0:
        out = {"coll": a.coll, "dtype": a.dtype, "n_gpus": d.world, "lib": a.lib or "nccl_b200", "symmetric": not a.plain, "rows": rows}
        text = json.dumps(out)
        print(text)
        if a.out:
            with open(a.out, "w") as f:
                f.write(text + "\n")


if __name__ == "__main__":
    main(sys.argv[1:])
