"""Times the tcgen05 GEMM kernels on one GPU (no communication) against cuBLAS.

    python -m nccl_b200.ops.tp_bench --dtype bf16 --shapes 8192x3584x8192,8192x8192x3584
    python -m nccl_b200.ops.tp_bench --dtype fp8  --shapes 8192x8192x8192 --iters 20

Shapes are MxNxK with C[M,N] = A[M,K] * W[N,K]^T. Inputs are larger than L2 for the default
shapes; timing is CUDA events around at least `iters` launches after a warm-up long enough to reach sustained
clocks (--warm-ms, --time-ms). Prints one line per shape.

Fused tensor-parallel layers (one process per GPU, torchrun), Llama-3-70B MLP shapes by default:

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m nccl_b200.ops.tp_bench --fused \
        --tokens 8192 --hidden 8192 --ffn 28672

times all-gather -> GEMM (column-parallel up projection) and GEMM -> reduce-scatter (row-parallel
down projection) in bf16 and block-scaled fp8, each against the unfused sequence (library
collective + cuBLAS GEMM; with --impl reference the collective comes from the reference build).
Prints one JSON line with times (max over ranks), TFLOP/s per GPU and the fraction of the
roofline max(FLOPs / bf16 GEMM peak, NVLink bytes / 770 GB/s) with the measured peaks of this pool.
"""
import argparse
import sys

import torch


def timed_sustained(fn, a, reduce_max, barrier):
    """Milliseconds per call of fn, CUDA events, max over ranks. A short burst runs at boost clocks and a long
    run at the power cap, 15-25 % apart on a dense GEMM, so every variant is first run for --warm-ms and then
    timed for at least --time-ms; the counts come from a 3-call estimate that all ranks agree on."""
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        fn()
    e1.record()
    torch.cuda.synchronize()
    est = max(reduce_max(e0.elapsed_time(e1) / 3), 1e-3)
    for _ in range(int(min(5000, a.warm_ms / est))):
        fn()
    torch.cuda.synchronize()
    barrier()
    iters = int(max(a.iters, min(5000, a.time_ms / est)))
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return reduce_max(e0.elapsed_time(e1) / iters)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="bf16", choices=("bf16", "fp8"))
    ap.add_argument("--shapes", default="8192x3584x8192,8192x8192x3584,8192x8192x8192")
    ap.add_argument("--iters", type=int, default=20, help="least number of timed launches")
    ap.add_argument("--warm-ms", type=float, default=400.0, help="warm every variant up for this long, so that all are timed at sustained (power-capped) clocks")
    ap.add_argument("--time-ms", type=float, default=300.0, help="time every variant for at least this long")
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--fused", action="store_true")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"), help="library of the unfused collectives")
    a = ap.parse_args(argv)
    if a.fused:
        return fused(a)
    from nccl_b200 import Communicator, get_unique_id
    from nccl_b200.ops.tp import TensorParallel
    torch.cuda.set_device(0)
    comm = Communicator(1, 0, get_unique_id())
    shapes = [tuple(int(v) for v in s.split("x")) for s in a.shapes.split(",")]
    tp = TensorParallel(comm, max(s[0] for s in shapes), max(s[1] for s in shapes))

    def timed(fn):
        return timed_sustained(fn, a, lambda v: v, lambda: None)

    for M, N, K in shapes:
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        flops = 2.0 * M * N * K
        if a.dtype == "fp8":
            xq, xs = tp.quantize_fp8(x, 1)
            wq, ws = tp.quantize_fp8(w, 128)
            ms = timed(lambda: tp.gemm_fp8(xq, xs, wq, ws, out=out))
            qms = timed(lambda: tp.quantize_fp8(x, 1, q=xq, scales=xs))
            extra = " | quantize activations %.3f ms (%.0f GB/s)" % (qms, M * K * 3 / qms / 1e6)
        else:
            ms = timed(lambda: tp.gemm(x, w, out=out))
            extra = ""
        line = "%s M%d N%d K%d: %.3f ms %.0f TFLOP/s" % (a.dtype, M, N, K, ms, flops / ms / 1e9)
        if not a.no_cublas:
            ref = timed(lambda: torch.matmul(x, w.t(), out=out))
            line += " | cuBLAS bf16 %.3f ms %.0f TFLOP/s" % (ref, flops / ref / 1e9)
        print(line + extra, flush=True)
        assert comm.async_error() == 0
    tp.destroy()
    comm.destroy()
    return 0


def fused(a):
    import json
    import os
    from nccl_b200 import Communicator, _lib, get_unique_id
    from nccl_b200.ops.tp import TensorParallel
    from nccl_b200.utils.perf import Dist
    d = Dist()
    torch.cuda.set_device(d.local_rank)
    n, rank = d.world, d.rank
    comm = Communicator(n, rank, d.bcast_bytes(get_unique_id() if rank == 0 else None))
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ref_path = os.path.join(root, "baseline", "_ref", "build", "lib", "libnccl.so.2")
    base = comm
    if a.impl == "reference":
        if not os.path.exists(ref_path):
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/build/lib/libnccl.so.2 is missing"}))
            return 0
        rl = _lib.load(ref_path)
        base = Communicator(n, rank, d.bcast_bytes(get_unique_id(rl) if rank == 0 else None), lib=rl)
    M, H, F = a.tokens, a.hidden, a.ffn
    Fl, Ml = F // n, M // n
    tp = TensorParallel(comm, M, max(H, Fl))
    g = torch.Generator(device="cuda").manual_seed(7 + rank)
    w_up = (torch.randn(Fl, H, device="cuda", generator=g) * 0.02).bfloat16()       # column-parallel: [F/n, H]
    w_dn = (torch.randn(H, Fl, device="cuda", generator=g) * 0.02).bfloat16()       # row-parallel:    [H, F/n]
    x_rows = torch.randn(Ml, H, device="cuda", generator=g).bfloat16()              # this rank's tokens
    act = torch.randn(M, Fl, device="cuda", generator=g).bfloat16()                 # input of the down projection
    xg = tp.alloc_gathered(M, H)
    xg[rank * Ml:(rank + 1) * Ml].copy_(x_rows)
    gq, gs = tp.alloc_gathered_fp8(M, H)
    mq, ms = tp.quantize_fp8(x_rows, 1)
    gq[rank * Ml:(rank + 1) * Ml].view(torch.uint8).copy_(mq.view(torch.uint8))
    gs[:, rank * Ml:(rank + 1) * Ml].copy_(ms)
    wq_up, ws_up = tp.quantize_fp8(w_up, 128)
    wq_dn, ws_dn = tp.quantize_fp8(w_dn, 128)
    aq, as_ = tp.quantize_fp8(act, 1)
    out_up = torch.empty(M, Fl, device="cuda", dtype=torch.bfloat16)
    out_dn = torch.empty(Ml, H, device="cuda", dtype=torch.bfloat16)
    full_dn = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    x_full = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    d.barrier()

    def timed(fn):
        return timed_sustained(fn, a, d.max, d.barrier)

    def unfused_up():
        base.all_gather(x_rows, x_full)
        torch.matmul(x_full, w_up.t(), out=out_up)

    def unfused_dn():
        torch.matmul(act, w_dn.t(), out=full_dn)
        base.reduce_scatter(full_dn, out_dn)

    t = {
        "ag_gemm_bf16": timed(lambda: tp.all_gather_gemm(xg, w_up, out=out_up)),
        "ag_gemm_fp8": timed(lambda: tp.all_gather_gemm_fp8(gq, wq_up, ws_up, out=out_up)),
        "gemm_rs_bf16": timed(lambda: tp.gemm_reduce_scatter(act, w_dn, out=out_dn)),
        "gemm_rs_fp8": timed(lambda: tp.gemm_reduce_scatter_fp8(aq, as_, wq_dn, ws_dn, out=out_dn)),
        "unfused_ag_then_gemm_bf16": timed(unfused_up),
        "unfused_gemm_then_rs_bf16": timed(unfused_dn),
    }
    assert comm.async_error() == 0
    flops = 2.0 * M * H * Fl
    peaks = {"bf16_tflops": 1590.0, "nvlink_gbs": 770.0}
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            mp = json.load(f)
        peaks["bf16_tflops"] = float(mp.get("bf16_tflops", peaks["bf16_tflops"]))
    except Exception:
        pass
    link_bytes = {"ag_gemm_bf16": (n - 1) * Ml * H * 2, "ag_gemm_fp8": (n - 1) * Ml * (H + H // 128 * 4),
                  "gemm_rs_bf16": (n - 1) * Ml * H * 4, "gemm_rs_fp8": (n - 1) * Ml * H * 4}
    res = {"metric": "tp_fused_ms", "impl_of_unfused_collectives": a.impl, "n_gpus": n, "tokens": M, "hidden": H, "ffn": F, "ms": {k: round(v, 4) for k, v in t.items()},
           "tflops_per_gpu": {k: round(flops / v / 1e9, 1) for k, v in t.items()}, "roofline_fraction": {}, "peaks": peaks}
    for k, b in link_bytes.items():
        ideal = max(flops / (peaks["bf16_tflops"] * 1e9), b / (peaks["nvlink_gbs"] * 1e6))
        res["roofline_fraction"][k] = round(ideal / t[k], 3)
    tp.destroy()
    if base is not comm:
        base.destroy()
    comm.destroy()
    if rank == 0:
        print(json.dumps(res), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
