#!/usr/bin/env python3
"""Turns measured performance data into a configuration file for the CSV tuner plugin (plugins/tuner/csv_tuner.cc).

Input: a CSV with the columns
    collective,size_bytes,algorithm,protocol,channels,nodes,ranks,pipeOps,regBuff[,cost_metric][,bandwidth_gbps][,latency_us]
one line per measurement of one (algorithm, protocol, channels) choice at one message size. For every collective and
topology (nodes, ranks, pipeOps, regBuff) the best choice per size is kept, neighbouring sizes with the same choice are merged,
and the borders between different choices are put at the geometric mean of the two sizes. Output lines have the form the plugin
reads:  collective,minBytes,maxBytes,algorithm,protocol,channels,nNodes,nRanks,numPipeOps,regBuff

    python plugins/tuner/optimize_config.py measurements.csv -o nccl_tuner.conf [-m latency_us] [--dry-run]

Reference parity: plugins/tuner/example/scripts/optimize_config.py (same input columns, metrics and options).
"""
import argparse
import csv
import math
import sys
from collections import defaultdict

METRICS = {"cost_metric": min, "latency_us": min, "bandwidth_gbps": max}   # which direction is better
REQUIRED = ["collective", "size_bytes", "algorithm", "protocol", "channels", "nodes", "ranks", "pipeOps", "regBuff"]


def read_rows(path, metric):
    with open(path, newline="") as f:
        reader = csv.DictReader(line for line in f if line.strip() and not line.lstrip().startswith("#"))
        missing = [c for c in REQUIRED if c not in (reader.fieldnames or [])]
        if missing:
            raise SystemExit("%s: missing column(s): %s" % (path, ", ".join(missing)))
        if metric not in (reader.fieldnames or []):
            raise SystemExit("%s: no column for the metric %s" % (path, metric))
        rows = []
        for n, row in enumerate(reader, 2):
            try:
                value = float(row[metric])
                size = int(row["size_bytes"])
            except (TypeError, ValueError):
                raise SystemExit("%s line %d: size_bytes and %s must be numbers" % (path, n, metric))
            rows.append((row["collective"].strip().lower(), int(row["nodes"]), int(row["ranks"]), int(row["pipeOps"]), int(row["regBuff"]), size,
                         (row["algorithm"].strip().lower(), row["protocol"].strip().lower(), int(row["channels"])), value))
    return rows


def optimise(rows, metric):
    """[(collective, lo, hi, algorithm, protocol, channels, nodes, ranks, pipeOps, regBuff)] in file order."""
    higher_is_better = METRICS[metric] is max
    best = defaultdict(dict)   # (collective, topology) -> size -> (value, choice)
    for coll, nodes, ranks, pipe, reg, size, choice, value in rows:
        slot = best[(coll, nodes, ranks, pipe, reg)]
        if size not in slot or (value > slot[size][0] if higher_is_better else value < slot[size][0]):
            slot[size] = (value, choice)
    out = []
    for (coll, nodes, ranks, pipe, reg), by_size in sorted(best.items()):
        sizes = sorted(by_size)
        runs = []          # [first size, last size, choice]
        for s in sizes:
            choice = by_size[s][1]
            if runs and runs[-1][2] == choice:
                runs[-1][1] = s
            else:
                runs.append([s, s, choice])
        for i, (first, last, choice) in enumerate(runs):
            lo = 0 if i == 0 else int(math.sqrt(runs[i - 1][1] * first)) + 1
            hi = (1 << 62) if i == len(runs) - 1 else int(math.sqrt(last * runs[i + 1][0]))
            out.append((coll, lo, hi, choice[0], choice[1], choice[2], nodes, ranks, pipe, reg))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description="best (algorithm, protocol, channels) per message size from measurements, as a CSV tuner configuration")
    ap.add_argument("input")
    ap.add_argument("-o", "--output", default="nccl_tuner.conf")
    ap.add_argument("-m", "--metric", default="cost_metric", choices=sorted(METRICS))
    ap.add_argument("--no-header", action="store_true")
    ap.add_argument("--dry-run", action="store_true", help="print the configuration instead of writing it")
    a = ap.parse_args(argv)
    rules = optimise(read_rows(a.input, a.metric), a.metric)
    lines = []
    if not a.no_header:
        lines += ["# made by optimize_config.py from %s (metric: %s)" % (a.input, a.metric),
                  "# collective,minBytes,maxBytes,algorithm,protocol,channels,nNodes,nRanks,numPipeOps,regBuff"]
    lines += [",".join(str(v) for v in r) for r in rules]
    text = "\n".join(lines) + "\n"
    if a.dry_run:
        sys.stdout.write(text)
    else:
        with open(a.output, "w") as f:
            f.write(text)
        print("%d rule(s) written to %s" % (len(rules), a.output))
    return 0


if __name__ == "__main__":
    sys.exit(main())
