"""Measures every algorithm variant of the data plane per collective and message size and derives
the crossover table that the library uses to pick a kernel (NCCL_TUNING_FILE format).

    torchrun --nproc-per-node N -m nccl_b200.utils.tune --out tuning_nN.json

For each (collective, size) it times: flagged lines (LL), peer loads/stores (P2P: push and pull
for the copy collectives), multimem (NVLS / MC), each at several CTA counts, on registered
symmetric buffers; device-timed, max over ranks. The selection the library makes by default is
then the fastest variant per size, expressed as thresholds.
"""
import argparse
import ctypes
import json
import sys

from .. import _lib
from ..core import BF16
from . import perf

ALGO_AUTO, ALGO_LL, ALGO_P2P, ALGO_NVLS = -1, 1, 2, 3
MODE_PUSH, MODE_PULL, MODE_MC = 0, 1, 2


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--limit", type=int, default=1 << 30, help="largest message in bytes")
    ap.add_argument("--colls", default="all_reduce,all_gather,reduce_scatter,all_to_all,broadcast")
    ap.add_argument("--ctas", default="8,16,32,64,128")
    ap.add_argument("--iters", type=int, default=30)
    a = ap.parse_args(argv)
    d = perf.Dist()
    lib = _lib.load()
    lib.b200ForceAlgo.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.b200ForceAlgo.restype = None
    lib.b200CommSetTuning.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_longlong]
    h = perf.Harness(d, lib, max_bytes=a.limit, symmetric=True)
    h.fill(BF16)
    n = d.world
    cta_list = [int(x) for x in a.ctas.split(",")]
    sizes = []
    s = 8
    while s <= a.limit:
        sizes.append(s)
        s *= 4
    if sizes[-1] != a.limit:
        sizes.append(a.limit)
    out = {"n_gpus": n, "results": {}}

    def set_ctas(c):
        for key in (b"nvlsCtas", b"p2pCtas", b"copyCtas"):
            lib.b200CommSetTuning(h.comm, key, 0, c)
        lib.b200CommSetTuning(h.comm, b"bytesPerCta", 0, 1)   # always use the cap

    def measure(coll, nb, algo, mode):
        lib.b200ForceAlgo(algo, mode)
        it = a.iters if nb <= (64 << 20) else 5
        try:
            return h.time(coll, nb, BF16, warmup=5 if nb <= (64 << 20) else 2, iters=it)
        finally:
            lib.b200ForceAlgo(ALGO_AUTO, -1)

    for coll in a.colls.split(","):
        res = {}
        div = n if coll in ("all_gather", "reduce_scatter", "all_to_all") else 1
        for nb0 in sizes:
            unit = 2 * div
            nb = max(unit, nb0 // unit * unit)
            block = nb // div   # bytes per rank block
            row = {}
            if block <= (1 << 20) - 8:
                row["LL"] = measure(coll, nb, ALGO_LL, -1)
            if block >= 1024:
                for c in cta_list:
                    set_ctas(c)
                    if coll in ("all_reduce", "reduce_scatter"):
                        row["P2P/%d" % c] = measure(coll, nb, ALGO_P2P, -1)
                        if block % 16 == 0:
                            row["NVLS/%d" % c] = measure(coll, nb, ALGO_NVLS, -1)
                    else:
                        row["PUSH/%d" % c] = measure(coll, nb, ALGO_P2P, MODE_PUSH)
                        row["PULL/%d" % c] = measure(coll, nb, ALGO_P2P, MODE_PULL)
                        if coll in ("all_gather", "broadcast") and block % 16 == 0:
                            row["MC/%d" % c] = measure(coll, nb, ALGO_NVLS, MODE_MC)
            best = min(row, key=row.get)
            factor = perf.bus_factor(coll, n)
            res[str(nb)] = {"best": best, "time_us": round(row[best], 2), "busbw_GBps": round(nb / row[best] / 1e3 * factor, 2),
                            "all": {k: round(v, 2) for k, v in row.items()}}
            if d.rank == 0:
                print("%s %d: best %s %.2f us busbw %.1f | %s" % (coll, nb, best, row[best], nb / row[best] / 1e3 * factor,
                                                                   " ".join("%s=%.1f" % kv for kv in sorted(row.items(), key=lambda kv: kv[1])[:5])), flush=True)
        out["results"][coll] = res
    h.close()
    if d.rank == 0:
        out["table"] = {str(n): {coll: rows_from(res) for coll, res in out["results"].items()}}
        print("TABLE " + json.dumps(out["table"]), flush=True)
        if a.out:
            with open(a.out, "w") as f:
                json.dump(out, f)


def rows_from(res):
    """[[upto_bytes, variant, ctas], ...]: the fastest variant per measured size, runs merged,
    each limit placed at the geometric mean of neighbouring sizes."""
    sizes = sorted(int(k) for k in res)
    rows = []
    for i, s in enumerate(sizes):
        best = res[str(s)]["best"]
        name, _, c = best.partition("/")
        upto = int((s * sizes[i + 1]) ** 0.5) if i + 1 < len(sizes) else 1 << 40
        row = [upto, name, int(c) if c else 0]
        if rows and rows[-1][1] == row[1] and rows[-1][2] == row[2]:
            rows[-1][0] = upto
        else:
            rows.append(row)
    return rows


if __name__ == "__main__":
    main(sys.argv[1:])
