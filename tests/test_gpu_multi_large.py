"""Messages above 4 GiB on two GPUs: byte offsets that do not fit 32 bits.

An all-reduce of 4 GiB + 16 bytes per rank and an all-gather of blocks of that size (so that the
second block starts 16 bytes past the 4 GiB mark of the output). Head, middle, the stretch around the
4 GiB boundary and the tail are compared with values recomputed from the fill pattern.
"""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402
from test_gpu_multi import _ngpus, _sym_tensor  # noqa: E402

pytestmark = pytest.mark.gpu

NUMEL = (1 << 30) + 4            # int32 elements: 4 GiB + 16 bytes


def _pattern(rank, lo, hi, device):
    """Element i of rank `rank`'s input: a value that depends on all bits of i."""
    import torch
    i = torch.arange(lo, hi, device=device, dtype=torch.int64)
    return ((i * 2654435761 + (i >> 20) * 97 + rank * 1000003) % 2000001 - 1000000).to(torch.int32)


def _large_rank(rank, nranks, uid):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    x = _sym_tensor(comm, NUMEL, torch.int32)
    y = _sym_tensor(comm, NUMEL * nranks, torch.int32)
    step = 1 << 27
    for lo in range(0, NUMEL, step):
        hi = min(NUMEL, lo + step)
        x[lo:hi] = _pattern(rank, lo, hi, "cuda")
    y.zero_()
    torch.cuda.synchronize()
    windows = [(0, 4096), (NUMEL // 2 - 2048, NUMEL // 2 + 2048), ((1 << 30) - 4096, NUMEL)]
    bad = []
    comm.all_reduce(x, y[:NUMEL])
    torch.cuda.synchronize()
    for lo, hi in windows:
        want = sum(_pattern(p, lo, hi, "cuda").to(torch.int64) for p in range(nranks)).to(torch.int32)
        if not torch.equal(y[lo:hi], want):
            bad.append(("all_reduce", lo, hi))
    y.zero_()
    torch.cuda.synchronize()
    comm.all_gather(x, y)
    torch.cuda.synchronize()
    for p in range(nranks):
        for lo, hi in windows:
            if not torch.equal(y[p * NUMEL + lo:p * NUMEL + hi], _pattern(p, lo, hi, "cuda")):
                bad.append(("all_gather", p, lo, hi))
    err = comm.async_error()
    comm.destroy()
    return {"bad": bad, "err": err}


def test_messages_above_four_gib():
    if _ngpus() < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_large_rank, 2, timeout=600)
    for r in range(2):
        assert res[r]["bad"] == [] and res[r]["err"] == 0, res[r]
