"""Data-parallel training step and ring attention through the library, on GPUs or on CPU ranks.

    # two CPU ranks (host-memory communicators over TCP), no GPU needed
    NCCL_B200_HOST_ONLY=1 python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/train_ddp_ring_attention.py
    # one rank per GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/train_ddp_ring_attention.py --device cuda

torch.distributed (gloo) only carries the unique id; all tensor traffic goes through nccl_b200.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from nccl_b200 import Communicator, get_unique_id  # noqa: E402
from nccl_b200.parallel.context import ring_attention  # noqa: E402
from nccl_b200.parallel.ddp import GradientBuckets  # noqa: E402
from nccl_b200.utils.perf import Dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu", choices=("cpu", "cuda"))
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args()
    d = Dist()
    if a.device == "cuda":
        torch.cuda.set_device(d.local_rank)
    else:
        os.environ.setdefault("NCCL_B200_HOST_ONLY", "1")
    comm = Communicator(d.world, d.rank, d.bcast_bytes(get_unique_id() if d.rank == 0 else None))

    # data parallel: same model everywhere, different data, averaged gradients
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 16)).to(a.device)
    buckets = GradientBuckets(comm, list(model.parameters()), bucket_bytes=16 << 10)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(1 + d.rank)
    x, y = torch.randn(32, 64, generator=g).to(a.device), torch.randn(32, 16, generator=g).to(a.device)
    losses = []
    for _ in range(a.steps):
        buckets.zero_grad()
        loss = ((model(x) - y) ** 2).mean()
        loss.backward()
        buckets.finish()
        opt.step()
        losses.append(float(loss))
    buckets.close()

    # context parallel: every rank holds a slice of the sequence
    gq = torch.Generator().manual_seed(7)
    q, k, v = [torch.randn(1, 4, 16 * d.world, 32, generator=gq) for _ in range(3)]
    sl = slice(d.rank * 16, (d.rank + 1) * 16)
    out = ring_attention(comm, *[t[:, :, sl].contiguous().to(a.device) for t in (q, k, v)], causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)[:, :, sl]
    err = float((out.cpu() - ref).abs().max())
    comm.destroy()
    print("rank %d: losses %s, ring attention max error %.2e" % (d.rank, " ".join("%.4f" % v for v in losses), err), flush=True)
    assert losses[-1] < losses[0] and err < 1e-3


if __name__ == "__main__":
    main()
