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

    _KINDS = {"all_reduce": (0, ("ncclAllReduce",)), "reduce_scatter": (0, ("ncclReduceScatter",)), "all_gather": (1, ("ncclAllGather",)),
              "all_to_all": (1, ("ncclAlltoAll",)), "broadcast": (2, ("ncclBroadcast",)), "reduce": (3, ("ncclReduce",)),
              "sendrecv": (4, ("ncclGroupStart", "ncclSend", "ncclRecv", "ncclGroupEnd"))}

    def _native_loop(self):
        """The loop of calls outside the interpreter (tools/perf_loop.c), or None when it is not built or switched off with
        NCCL_B200_PERF_PYTHON_LOOP=1. It gets the entry points of the library under test as addresses."""
        if not hasattr(self, "_loop"):
            self._loop = None
            path = os.path.join(os.path.dirname(_lib.LIB_PATH), "libperf_loop.so")
            if os.environ.get("NCCL_B200_PERF_PYTHON_LOOP", "0") != "1" and os.path.exists(path):
                try:
                    fn = ctypes.CDLL(path).perfLoop
                    fn.restype = ctypes.c_int
                    fn.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
                    self._loop = fn
                except (OSError, AttributeError):
                    self._loop = None
        return self._loop

    def calls(self, coll, nbytes, dtype_code, stream_ptr, iters):
        """Issues `iters` calls of one collective back to back; returns the first result that is not ncclSuccess, else 0."""
        loop = self._native_loop()
        if loop is not None and coll in self._KINDS:
            kind, names = self._KINDS[coll]
            key = (coll,)
            if not hasattr(self, "_fns"):
                self._fns = {}
            if key not in self._fns:
                self._fns[key] = (ctypes.c_void_p * len(names))(*[ctypes.cast(getattr(self.lib, nm), ctypes.c_void_p).value for nm in names])
            es = TYPE_SIZE[dtype_code]
            count = nbytes // es // (self.n if coll in ("all_gather", "reduce_scatter", "all_to_all") else 1)
            comm = self.comm if isinstance(self.comm, ctypes.c_void_p) else ctypes.c_void_p(getattr(self.comm, "value", self.comm))
            return loop(kind, self._fns[key], self.send_ptr, self.recv_ptr, count, dtype_code, 0, 0, (self.rank + 1) % self.n, (self.rank - 1) % self.n,
                        comm, stream_ptr, iters)
        for _ in range(iters):
            r = self.call(coll, nbytes, dtype_code, stream_ptr)
            if r != 0:
                return r
        return 0

    def time(self, coll, nbytes, dtype_code=FP32, warmup=20, iters=100, min_warm_ms=3.0, passes=2):
        """Mean device time per call in microseconds (max over ranks). The warm-up covers at least
        `warmup` calls and roughly `min_warm_ms` of device time: after the host-side barrier between
        two measurements the GPU has been idle and its clocks have dropped, and a window of a few
        short kernels would otherwise be timed at idle clocks. The number of warm-up calls is a
        function of the message size only, so every rank issues the same sequence of collectives."""
        sp = self.stream.cuda_stream
        est_us = 10.0 + nbytes / 3.0e5                       # rough per-call time: 10 us + bytes at 300 GB/s
        warm = max(warmup, min(2000, int(min_warm_ms * 1e3 / est_us) + 1))
        # The host issues the calls while the device runs them, so a pause of the interpreter (a
        # garbage-collection pass takes milliseconds) would be timed as if it were the library's:
        # collection is off inside the loop, and the loop runs twice with the faster pass reported.
        import gc
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.stream(self.stream):
                self.d.barrier()
                _lib.check(self.calls(coll, nbytes, dtype_code, sp, warm), coll, self.lib)
                self.stream.synchronize()
                best = None
                for _ in range(passes):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(self.stream)
                    _lib.check(self.calls(coll, nbytes, dtype_code, sp, iters), coll, self.lib)
                    e1.record(self.stream)
                    self.stream.synchronize()
                    us = e0.elapsed_time(e1) * 1000.0 / iters
                    best = us if best is None else min(best, us)
        finally:
            if was_enabled:
                gc.enable()
        return self.d.max(best)

    def time_host(self, coll, nbytes, dtype_code=FP32, iters=200):
        """Host time per call in microseconds (max over ranks): how long the calling thread spends
        inside the library per collective while the device queue is not full."""
        import time as _time
        sp = self.stream.cuda_stream
        with torch.cuda.stream(self.stream):
            self.d.barrier()
            _lib.check(self.calls(coll, nbytes, dtype_code, sp, 20), coll, self.lib)
            self.stream.synchronize()
            t0 = _time.perf_counter()
            self.calls(coll, nbytes, dtype_code, sp, iters)
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


class Verifier:
    """Checks results on the device against values recomputed from the seeds of all ranks.

    Every rank can regenerate every other rank's input (Harness.fill draws from a generator seeded
    with 7 + rank in chunks of 2^26 elements), so no data has to travel: the verifier keeps the
    first `prefix_bytes` of every rank's input and, for messages that reach further, regenerates on
    demand. A check runs the collective once, then compares windows of the output (the whole output
    when it is small; otherwise the head, the tail and a stretch around every block boundary) with a
    plain PyTorch fp32 computation. Nothing of this is inside a timed region."""

    def __init__(self, h, dtype_code, prefix_bytes):
        self.h = h
        self.dt = dtype_code
        self.tdt = torch.bfloat16 if dtype_code == BF16 else torch.float32
        self.es = TYPE_SIZE[dtype_code]
        self.prefix = min(prefix_bytes, h.max_bytes) // self.es
        self._chunk_states = {}
        self.inputs = [self._regen(p, self.prefix) for p in range(h.n)]
        self.max_err = 0.0
        self.points = 0
        self.failures = []

    def _states(self, p):
        """Generator state of rank p before each 2^26-element chunk (one pass over the whole buffer, once)."""
        if p not in self._chunk_states:
            g = torch.Generator(device="cuda").manual_seed(7 + p)
            total = self.h.send_bytes // self.es
            states = []
            for i in range(0, total, 1 << 26):
                states.append(g.get_state())
                torch.rand(min(1 << 26, total - i), generator=g, device="cuda", dtype=torch.float32)
            self._chunk_states[p] = states
        return self._chunk_states[p]

    def _regen(self, p, numel, skip=0):
        """Elements [skip, skip + numel) of rank p's input, drawn exactly as Harness.fill draws them."""
        total = self.h.send_bytes // self.es
        step = 1 << 26
        states = self._states(p)
        g = torch.Generator(device="cuda")
        parts = []
        for ci in range(skip // step, (skip + numel - 1) // step + 1):
            i = ci * step
            m = min(step, total - i)
            g.set_state(states[ci])
            chunk = (torch.rand(m, generator=g, device="cuda", dtype=torch.float32) * 2 - 1).to(self.tdt)
            lo, hi = max(skip, i), min(skip + numel, i + m)
            parts.append(chunk[lo - i:hi - i].clone())
            del chunk
        return torch.cat(parts) if len(parts) != 1 else parts[0]

    def _src(self, p, lo, hi):
        if hi <= self.prefix:
            return self.inputs[p][lo:hi]
        return self._regen(p, hi - lo, lo)

    @staticmethod
    def _windows(numel, edge=1 << 11, whole=1 << 22):
        if numel <= whole:
            return [(0, numel)]
        return [(0, min(numel, 1 << 20)), (numel // 2 - edge, numel // 2 + edge), (numel - edge, numel)]

    def _cmp(self, got, want, exact, what):
        if exact:
            ok = torch.equal(got, want)
            err = 0.0 if ok else float((got.float() - want.float()).abs().max())
        else:
            # sums of n values of magnitude <= 1: fp32 accumulation, one rounding to the element type
            eps = 2.0 ** -7 if self.tdt == torch.bfloat16 else 2.0 ** -20
            diff = (got.float() - want).abs()
            err = float(diff.max()) if diff.numel() else 0.0
            ok = bool((diff <= eps * (1.0 + want.abs())).all())
        self.max_err = max(self.max_err, err)
        if not ok:
            self.failures.append("%s: max abs error %.4g" % (what, err))
        return ok

    def check(self, coll, nbytes):
        """Runs `coll` once at this size and checks the output. Returns True when it is right."""
        h, n, r, es = self.h, self.h.n, self.h.rank, self.es
        unit = es * (n if coll in ("all_gather", "reduce_scatter", "all_to_all") else 1)
        nb = max(unit, nbytes // unit * unit)
        out = h.recv_t.view(self.tdt)
        out[: max(nb // es, 1)].zero_()
        torch.cuda.synchronize()
        with torch.cuda.stream(h.stream):
            _lib.check(h.call(coll, nb, self.dt, h.stream.cuda_stream), coll, h.lib)
        torch.cuda.synchronize()
        ok = True
        tag = "%s %d B rank %d" % (coll, nb, r)
        if coll in ("all_reduce", "reduce"):
            if coll == "reduce" and r != 0:
                return True
            for lo, hi in self._windows(nb // es):
                want = torch.zeros(hi - lo, dtype=torch.float32, device="cuda")
                for p in range(n):
                    want += self._src(p, lo, hi).float()
                ok &= self._cmp(out[lo:hi], want, False, tag)
        elif coll == "reduce_scatter":
            blk = nb // es // n
            for lo, hi in self._windows(blk):
                want = torch.zeros(hi - lo, dtype=torch.float32, device="cuda")
                for p in range(n):
                    want += self._src(p, r * blk + lo, r * blk + hi).float()
                ok &= self._cmp(out[lo:hi], want, False, tag)
        elif coll == "all_gather":
            blk = nb // es // n
            for p in range(n):
                for lo, hi in self._windows(blk, whole=1 << 19):
                    ok &= self._cmp(out[p * blk + lo:p * blk + hi], self._src(p, lo, hi), True, tag)
        elif coll == "all_to_all":
            blk = nb // es // n
            for p in range(n):
                for lo, hi in self._windows(blk, whole=1 << 19):
                    ok &= self._cmp(out[p * blk + lo:p * blk + hi], self._src(p, r * blk + lo, r * blk + hi), True, tag)
        elif coll == "broadcast":
            for lo, hi in self._windows(nb // es):
                ok &= self._cmp(out[lo:hi], self._src(0, lo, hi), True, tag)
        elif coll == "sendrecv":
            for lo, hi in self._windows(nb // es):
                ok &= self._cmp(out[lo:hi], self._src((r - 1) % n, lo, hi), True, tag)
        self.points += 1
        return ok

    def summary(self):
        """Agreed over all ranks: {"ok", "points", "max_err", "failures"}."""
        bad = self.h.d.max(float(len(self.failures)))
        return {"ok": bad == 0, "points": self.points, "max_abs_err": self.h.d.max(self.max_err), "failures": self.failures[:4]}


def sweep(h, coll, dtype_code, sizes, warmup=20, iters=100, verifier=None):
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
        row = {"bytes": nb, "time_us": round(us, 2), "algbw_GBps": round(alg, 2), "busbw_GBps": round(alg * bus_factor(coll, h.n), 2)}
        if verifier is not None:
            row["verified"] = verifier.check(coll, nb)
        rows.append(row)
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
    ap.add_argument("--verify", action="store_true", help="check every size against values recomputed from the seeds (outside the timed loops)")
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
        ver = Verifier(h, dt, min(a.max, 256 << 20)) if a.verify else None
        rows = sweep(h, a.coll, dt, sizes, a.warmup, a.iters, ver)
    verified = ver.summary() if (not a.latency and ver is not None) else None
    h.close()
    if d.rank == 0:
        out = {"coll": a.coll, "dtype": a.dtype, "n_gpus": d.world, "lib": a.lib or "nccl_b200", "symmetric": not a.plain, "rows": rows}
        if verified is not None:
            out["verified"] = verified
        text = json.dumps(out)
        print(text)
        if a.out:
            with open(a.out, "w") as f:
                f.write(text + "\n")


if __name__ == "__main__":
    main(sys.argv[1:])
