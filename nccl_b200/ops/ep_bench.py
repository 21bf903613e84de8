"""Expert-parallel dispatch / combine benchmark (one process per GPU, launched with torchrun).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m nccl_b200.ops.ep_bench \
        --tokens 4096 --hidden 7168 --experts 256 --topk 8 --iters 20

Routing: top-k of a softmax over N(0,1) logits (skewed loads). Dispatch sends e4m3 tokens with one
fp32 scale per 128 values; combine returns bf16 and applies the gate weights. Times are CUDA events,
max over ranks; bandwidth counts the bytes a rank receives (dispatch) or sends back (combine).
--baseline also times the unfused sequence on the stock collective library through
torch.distributed: sort by destination + quantise + all_to_all_single, and the reverse for combine.
"""
import argparse
import json
import os
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--baseline", action="store_true")
    ap.add_argument("--layout", default="expert_major", choices=["expert_major", "rank_major", "flat"],
                    help="rank_major / flat: one copy of a token per destination rank instead of one per selected expert")
    ap.add_argument("--phases", action="store_true", help="also time the sending and the receiving half of each call on their own (send_only + complete)")
    a = ap.parse_args(argv)
    from nccl_b200 import Communicator, get_unique_id
    from nccl_b200.ops.ep import ExpertParallel
    from nccl_b200.utils.perf import Dist
    d = Dist()
    torch.cuda.set_device(d.local_rank)
    n, rank = d.world, d.rank
    uid = d.bcast_bytes(get_unique_id() if rank == 0 else None)
    comm = Communicator(n, rank, uid)
    T, H, E, K = a.tokens, a.hidden, a.experts, a.topk
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    logits = torch.randn(T, E, device="cuda", generator=g)
    w, idx = torch.softmax(logits, -1).topk(K, dim=-1)
    w = (w / w.sum(-1, keepdim=True)).float().contiguous()
    idx = idx.long().contiguous()
    ep = ExpertParallel(comm, E, T, H, layout=a.layout)
    El, cap = E // n, n * T
    lead = {"expert_major": (El, cap), "rank_major": (n, T), "flat": (cap,)}[a.layout]
    toks = torch.empty(*lead, H, dtype=torch.uint8, device="cuda")
    scales = torch.empty(*lead, H // 128, dtype=torch.float32, device="cuda")
    counts = torch.zeros(El, dtype=torch.int32, device="cuda")
    y = torch.empty(*lead, H, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")

    def timed(fn, sync_before=None):
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        d.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return d.max(e0.elapsed_time(e1) / a.iters)

    disp_ms = timed(lambda: ep.dispatch(x, idx, w, fp8=True, toks=toks, scales=scales, counts=counts))
    ep.dispatch(x, idx, w, fp8=True, toks=toks, scales=scales, counts=counts)
    torch.cuda.synchronize()
    # rows that crossed: one per (token, selected expert) or, for the per-rank layouts, one per (token, destination rank)
    recv_tokens = int(counts.sum().item()) if a.layout == "expert_major" else int((ep.recv_topk_idx >= 0).any(-1).sum().item())
    y.zero_()
    comb_ms = timed(lambda: ep.combine(y, out=out))
    both_ms = timed(lambda: (ep.dispatch(x, idx, w, fp8=True, toks=toks, scales=scales, counts=counts), ep.combine(y, out=out)))
    phases = None
    if a.phases:
        # The halves of a call as two kernels: when their sum is far below the time of the whole call, the two sides get in each
        # other's way inside one kernel (e.g. receivers polling while rows still arrive), not the copies themselves.
        def halves(first):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            s_us, r_us = [], []
            for _ in range(a.warmup + a.iters):
                if first is ep.combine:
                    ep.dispatch(x, idx, w, fp8=True, toks=toks, scales=scales, counts=counts)
                torch.cuda.synchronize()
                d.barrier()
                ev[0].record()
                if first is ep.combine:
                    ep.combine(y, out=out, send_only=True)
                else:
                    ep.dispatch(x, idx, w, fp8=True, toks=toks, scales=scales, counts=counts, send_only=True)
                ev[1].record()
                ep.complete()
                ev[2].record()
                torch.cuda.synchronize()
                s_us.append(ev[0].elapsed_time(ev[1]) * 1e3)
                r_us.append(ev[1].elapsed_time(ev[2]) * 1e3)
            k = a.warmup
            return d.max(sum(s_us[k:]) / len(s_us[k:])), d.max(sum(r_us[k:]) / len(r_us[k:]))
        ds, dr = halves(ep.dispatch)
        cs, cr = halves(ep.combine)
        phases = {"dispatch_send_us": ds, "dispatch_receive_us": dr, "combine_send_us": cs, "combine_receive_us": cr}
    recv_max = d.max(float(recv_tokens))
    res = {"metric": "ep_dispatch_combine", "layout": a.layout, "n_gpus": n, "tokens_per_rank": T, "hidden": H, "experts": E, "topk": K,
           "dispatch_us": disp_ms * 1e3, "combine_us": comb_ms * 1e3, "dispatch_plus_combine_us": both_ms * 1e3,
           "recv_tokens_max": int(recv_max),
           "dispatch_GBps": recv_max * (H + H // 128 * 4) / disp_ms / 1e6, "combine_GBps": recv_max * H * 2 / comb_ms / 1e6}
    # Roofline: the bytes the busiest rank must receive (dispatch) or return (combine), of which (n - 1) / n cross NVLink,
    # over the measured peer-copy bandwidth per direction per GPU.
    link = 770.0
    res["roofline_fraction"] = {"dispatch": round(res["dispatch_GBps"] * (n - 1) / n / link, 3) if n > 1 else None,
                                "combine": round(res["combine_GBps"] * (n - 1) / n / link, 3) if n > 1 else None}
    res["peaks"] = {"nvlink_gbs": link}
    if phases is not None:
        res["phases"] = phases
    assert comm.async_error() == 0
    ep.destroy()

    if a.baseline and n > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_PORT", "29512")
        pg = dist.new_group(backend="nccl")
        dest = idx // El                                        # destination rank of every (token, k)
        order = torch.argsort(dest.view(-1), stable=True)
        send_counts = torch.bincount(dest.view(-1), minlength=n)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=pg)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        tok_of = (order // K)

        def base_dispatch():
            xs = x[tok_of]                                      # permute (gather rows)
            amax = xs.float().view(-1, H // 128, 128).abs().amax(-1).clamp_min(1e-10)
            sc_ = amax / 448.0
            q = (xs.float().view(-1, H // 128, 128) / sc_.unsqueeze(-1)).to(torch.float8_e4m3fn).view(-1, H)
            rq = torch.empty(sum(rc), H, dtype=torch.uint8, device="cuda")
            rs = torch.empty(sum(rc), H // 128, dtype=torch.float32, device="cuda")
            dist.all_to_all_single(rq, q.view(torch.uint8), rc, sc, group=pg)
            dist.all_to_all_single(rs, sc_, rc, sc, group=pg)
            return rq, rs

        rq, _ = base_dispatch()
        yb = torch.zeros(rq.shape[0], H, dtype=torch.bfloat16, device="cuda")

        def base_combine():
            back = torch.empty(T * K, H, dtype=torch.bfloat16, device="cuda")
            dist.all_to_all_single(back, yb, sc, rc, group=pg)
            full = torch.empty_like(back)
            full[order] = back
            return (full.view(T, K, H).float() * w.unsqueeze(-1)).sum(1).bfloat16()

        res["baseline_dispatch_us"] = timed(base_dispatch) * 1e3
        res["baseline_combine_us"] = timed(base_combine) * 1e3
        res["baseline"] = "torch.distributed (stock library) all_to_all_single + separate permute / quantise / weighted-sum kernels"
    comm.destroy()
    if rank == 0:
        print(json.dumps(res), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
