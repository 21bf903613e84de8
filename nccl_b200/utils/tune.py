"""Measures every algorithm variant of the data plane per collective and message size and derives
the selection table that the library uses to pick a kernel (NCCL_TUNING_FILE format).

    torchrun --nproc-per-node N -m nccl_b200.utils.tune --out tuning_nN.json

For each (collective, size) it times: flagged lines (LL), peer loads/stores (P2P: push and pull
for the copy collectives), multimem (NVLS two-shot, NVLS1 one-shot all-reduce, MC copies), the copy collectives also moved by
the bulk-copy engines (BPUSH / BPULL / BMC: few CTAs), each at several CTA counts, on registered symmetric buffers; device-timed, max over ranks. Two switches
that are global per rank count are measured as well: publishing flagged lines with one multimem.st
("+mc" variants) and arriving at barriers with one multimem.red ("+mb" variants); each is turned
on when the variants it affects are faster with it on average. The table then takes, per size, the
fastest variant, and among CTA counts of that variant the smallest one within `--slack` of it:
SMs not taken by a collective stay with the compute kernels it overlaps.
"""
import argparse
import ctypes
import json
import math
import time
import sys

from .. import _lib
from ..core import BF16, FP32
from . import perf

ALGO_AUTO, ALGO_LL, ALGO_P2P, ALGO_NVLS, ALGO_CE, ALGO_NVLS1 = -1, 1, 2, 3, 6, 8
MODE_PUSH, MODE_PULL, MODE_MC, MODE_SPLIT, MODE_BULK = 0, 1, 2, 3, 4


def size_list(limit, fine_lo=64 << 10, fine_hi=128 << 20):
    """x4 steps from 8 bytes, x2 between fine_lo and fine_hi where the crossovers are."""
    sizes, s = [], 8
    while s <= limit:
        sizes.append(s)
        s *= 2 if fine_lo <= s < fine_hi else 4
    if sizes[-1] != limit:
        sizes.append(limit)
    return sizes


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--table-out", default=None, help="write only the selection table here (a file NCCL_TUNING_FILE accepts)")
    ap.add_argument("--limit", type=int, default=1 << 30, help="largest message in bytes")
    ap.add_argument("--colls", default="all_reduce,all_gather,reduce_scatter,all_to_all,broadcast")
    ap.add_argument("--ctas", default="2,4,8,16,32,64,128")
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--dtype", default="bf16", choices=("bf16", "fp32"))
    ap.add_argument("--slack", type=float, default=0.03, help="prefer the smallest CTA count within this fraction of the fastest")
    ap.add_argument("--budget", type=float, default=0, help="seconds after which no further size is started (0 = no limit); the table is made from what was measured")
    ap.add_argument("--toggles", default="auto", choices=("auto", "off"), help="auto: also measure the multimem barrier / flagged-line switches when multicast is available")
    a = ap.parse_args(argv)
    d = perf.Dist()
    lib = _lib.load()
    lib.b200ForceAlgo.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.b200ForceAlgo.restype = None
    lib.b200CommSetTuning.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_longlong]
    lib.b200CommHasMulticast.argtypes = [ctypes.c_void_p]
    h = perf.Harness(d, lib, max_bytes=a.limit, symmetric=True)
    dt = BF16 if a.dtype == "bf16" else FP32
    h.fill(dt)
    n = d.world
    has_mc = bool(lib.b200CommHasMulticast(h.comm)) and a.toggles == "auto"
    cta_list = [int(x) for x in a.ctas.split(",")]
    sizes = size_list(a.limit)
    out = {"n_gpus": n, "dtype": a.dtype, "results": {}}

    def set_ctas(c):
        for key in (b"nvlsCtas", b"p2pCtas", b"copyCtas"):
            lib.b200CommSetTuning(h.comm, key, 0, c)
        lib.b200CommSetTuning(h.comm, b"bytesPerCta", 0, 1)   # always use the cap

    def toggles(mb, mc):
        lib.b200CommSetTuning(h.comm, b"barrierMcMin", 0, 2 if mb else 0)
        lib.b200CommSetTuning(h.comm, b"llMcMin", 0, 2 if mc else 0)

    def measure(coll, nb, algo, mode):
        lib.b200ForceAlgo(algo, mode)
        big = nb > (64 << 20)
        try:
            return h.time(coll, nb, dt, warmup=2 if big else 5, iters=5 if big else a.iters)
        finally:
            lib.b200ForceAlgo(ALGO_AUTO, -1)

    t_start = time.time()
    stopped = False
    for coll in a.colls.split(","):
        if stopped:
            break
        res = {}
        div = n if coll in ("all_gather", "reduce_scatter", "all_to_all") else 1
        reduces = coll in ("all_reduce", "reduce_scatter")
        for nb0 in sizes:
            # every rank takes the same decision: the slowest clock counts
            if a.budget and d.max(time.time() - t_start) > a.budget:
                stopped = True
                break
            unit = 2 * div
            nb = max(unit, nb0 // unit * unit)
            block = nb // div   # bytes per rank block
            row = {}
            if block <= (1 << 20) - 8:
                toggles(False, False)
                row["LL"] = measure(coll, nb, ALGO_LL, -1)
                if has_mc and coll in ("all_reduce", "all_gather"):
                    toggles(False, True)
                    row["LL+mc"] = measure(coll, nb, ALGO_LL, -1)
            if block >= 1024:
                for c in cta_list:
                    # a CTA of 512 threads moves 8 KiB per round: more CTAs than rounds only add barrier traffic
                    if c > cta_list[0] and block < c * 4096:
                        continue
                    set_ctas(c)
                    for mb in ((False, True) if has_mc else (False,)):
                        toggles(mb, False)
                        sfx = "+mb" if mb else ""
                        if reduces:
                            if n <= 2 or block >= (256 << 10):
                                row["P2P/%d%s" % (c, sfx)] = measure(coll, nb, ALGO_P2P, -1)
                            if block % 16 == 0:
                                row["NVLS/%d%s" % (c, sfx)] = measure(coll, nb, ALGO_NVLS, -1)
                                if coll == "all_reduce" and nb <= (4 << 20) and c <= 32:
                                    row["NVLS1/%d%s" % (c, sfx)] = measure(coll, nb, ALGO_NVLS1, -1)
                        else:
                            row["PUSH/%d%s" % (c, sfx)] = measure(coll, nb, ALGO_P2P, MODE_PUSH)
                            row["PULL/%d%s" % (c, sfx)] = measure(coll, nb, ALGO_P2P, MODE_PULL)
                            if coll in ("all_gather", "broadcast") and block % 16 == 0:
                                row["MC/%d%s" % (c, sfx)] = measure(coll, nb, ALGO_NVLS, MODE_MC)
                            # bulk-copy engines: worth it where a CTA has several 32 KiB chunks to stream
                            if block % 16 == 0 and block >= c * (64 << 10) and c <= 32:
                                row["BPUSH/%d%s" % (c, sfx)] = measure(coll, nb, ALGO_P2P, MODE_PUSH | MODE_BULK)
                                row["BPULL/%d%s" % (c, sfx)] = measure(coll, nb, ALGO_P2P, MODE_PULL | MODE_BULK)
                                if coll in ("all_gather", "broadcast"):
                                    row["BMC/%d%s" % (c, sfx)] = measure(coll, nb, ALGO_NVLS, MODE_MC | MODE_BULK)
                            # broadcast shared out among the non-root ranks: worth it where the root's store stream is the limit
                            if coll == "broadcast" and n >= 3 and block % 16 == 0 and block >= (1 << 20):
                                row["SPLIT/%d%s" % (c, sfx)] = measure(coll, nb, ALGO_P2P, MODE_SPLIT)
            toggles(False, False)
            if not reduces and coll != "broadcast" and nb >= (1 << 20):
                row["CE"] = measure(coll, nb, ALGO_CE, -1)   # copy engines: zero SMs
            best = min(row, key=row.get)
            factor = perf.bus_factor(coll, n)
            res[str(nb)] = {"best": best, "time_us": round(row[best], 2), "busbw_GBps": round(nb / row[best] / 1e3 * factor, 2),
                            "all": {k: round(v, 2) for k, v in row.items()}}
            if d.rank == 0:
                print("%s %d: best %s %.2f us busbw %.1f | %s" % (coll, nb, best, row[best], nb / row[best] / 1e3 * factor,
                                                                   " ".join("%s=%.1f" % kv for kv in sorted(row.items(), key=lambda kv: kv[1])[:6])), flush=True)
        out["results"][coll] = res
        if d.rank == 0 and a.out:   # kept up to date: a run that is cut short still leaves what it measured
            with open(a.out, "w") as f:
                json.dump(out, f)
    h.close()
    if d.rank == 0:
        use_mc, use_mb = decide_toggles(out["results"])
        out["toggles"] = {"llMc": use_mc, "barrierMc": use_mb}
        table = {coll: rows_from(res, use_mc, use_mb, a.slack) for coll, res in out["results"].items()}
        out["table"] = {str(n): table, "llMcMin": n if use_mc else 0, "barrierMcMin": n if use_mb else 0}
        print("TOGGLES " + json.dumps(out["toggles"]), flush=True)
        print("TABLE " + json.dumps(out["table"]), flush=True)
        if a.out:
            with open(a.out, "w") as f:
                json.dump(out, f)
        if a.table_out:
            with open(a.table_out, "w") as f:
                json.dump(out["table"], f)


def _split(name):
    """'NVLS/8+mb' -> ('NVLS', 8, 'mb'); 'LL+mc' -> ('LL', 0, 'mc')."""
    base, _, tog = name.partition("+")
    algo, _, c = base.partition("/")
    return algo, int(c) if c else 0, tog


def decide_toggles(results):
    """A switch is on when the best time over the variants it affects is lower with it, in the
    geometric mean over all measured points."""
    def gain(tog):
        logs = []
        for res in results.values():
            for cell in res.values():
                on = [t for k, t in cell["all"].items() if _split(k)[2] == tog]
                # "mc" changes the flagged-line kernels, "mb" every kernel that uses barriers
                off = [t for k, t in cell["all"].items() if _split(k)[2] == "" and (_split(k)[0] == "LL") == (tog == "mc")]
                if on and off:
                    logs.append(math.log(min(off) / min(on)))
        return math.exp(sum(logs) / len(logs)) if logs else 0.0
    return gain("mc") > 1.01, gain("mb") > 1.01


def rows_from(res, use_mc=False, use_mb=False, slack=0.03):
    """[[upto_bytes, variant, ctas], ...]: per measured size the fastest variant under the chosen
    switches (smallest CTA count within `slack` of it), runs merged, each limit placed at the
    geometric mean of neighbouring sizes."""
    sizes = sorted(int(k) for k in res)
    rows = []
    for i, s in enumerate(sizes):
        cand = {}
        plain = {}
        for k, t in res[str(s)]["all"].items():
            algo, c, tog = _split(k)
            want = ("mc" if use_mc else "") if algo == "LL" else ("mb" if use_mb else "")
            if tog == want:
                cand[(algo, c)] = t
            if tog == "":
                plain[(algo, c)] = t
        for key, t in plain.items():   # variants that the switch does not change (no "+mc" / "+mb" twin was measured)
            cand.setdefault(key, t)
        (algo, c), tbest = min(cand.items(), key=lambda kv: kv[1])
        if ("CE", 0) in cand and cand[("CE", 0)] <= tbest * (1 + slack):
            algo, c = "CE", 0                      # as fast as the best kernel and takes no SM
        else:
            frugal = [cc for (aa, cc), t in cand.items() if aa == algo and t <= tbest * (1 + slack)]
            c = min(frugal)
        upto = int((s * sizes[i + 1]) ** 0.5) if i + 1 < len(sizes) else 1 << 40
        row = [upto, algo, c]
        if rows and rows[-1][1] == row[1] and rows[-1][2] == row[2]:
            rows[-1][0] = upto
        else:
            rows.append(row)
    return rows


if __name__ == "__main__":
    main(sys.argv[1:])
