"""Real multi-GPU runs: one process per GPU, collectives through the public API.

Skipped unless the machine has at least two GPUs. Every case checks against a PyTorch reference
computed from the seeds of all ranks.
"""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu


def _ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _sym_tensor(comm, numel, dtype):
    """A tensor over ncclMemAlloc memory registered as a symmetric window of `comm`."""
    import torch
    from nccl_b200 import mem_alloc
    from nccl_b200.utils.perf import tensor_at
    es = torch.empty(0, dtype=dtype).element_size()
    nbytes = max(numel * es, 16)
    ptr = mem_alloc(nbytes)
    t = tensor_at(ptr, nbytes)[:numel * es].view(dtype)
    comm.register_window(tensor_at(ptr, nbytes))
    return t


def _inputs(rank, numel, dtype, seed=100):
    import torch
    g = torch.Generator().manual_seed(seed + rank)
    if dtype.is_floating_point:
        return torch.randn(numel, generator=g).to(dtype)
    return torch.randint(-50, 50, (numel,), generator=g).to(dtype)


def _colls_rank(rank, nranks, uid, registered, algo):
    import os
    import torch
    if algo:
        os.environ["NCCL_ALGO"] = algo
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator, group
    comm = Communicator(nranks, rank, uid)
    n = nranks
    res = {}

    def buf(numel, dtype):
        return _sym_tensor(comm, numel, dtype) if registered else torch.empty(numel, dtype=dtype, device="cuda")

    for dtype, numel in ((torch.float32, 1 << 20), (torch.bfloat16, (1 << 18) + 8), (torch.float32, 257), (torch.int32, 5000), (torch.bfloat16, 64)):
        x = buf(numel, dtype)
        y = buf(numel, dtype)
        x.copy_(_inputs(rank, numel, dtype))
        for op in ("sum", "max"):
            comm.all_reduce(x, y, op=op)
            torch.cuda.synchronize()
            res[("ar", str(dtype), numel, op)] = y.cpu()
    # all-gather / reduce-scatter / all-to-all / broadcast
    per = 4096 + 16
    s = buf(per, torch.float32)
    s.copy_(_inputs(rank, per, torch.float32, 7))
    g = buf(per * n, torch.float32)
    comm.all_gather(s, g)
    torch.cuda.synchronize()
    res["ag"] = g.cpu()
    big = buf(per * n, torch.float32)
    big.copy_(_inputs(rank, per * n, torch.float32, 9))
    rs = buf(per, torch.float32)
    comm.reduce_scatter(big, rs)
    torch.cuda.synchronize()
    res["rs"] = rs.cpu()
    a2a = buf(per * n, torch.float32)
    comm.all_to_all(big, a2a)
    torch.cuda.synchronize()
    res["a2a"] = a2a.cpu()
    b = buf(1000, torch.float32)
    b.copy_(_inputs(rank, 1000, torch.float32, 11))
    comm.broadcast(b, b, root=n - 1)
    torch.cuda.synchronize()
    res["bc"] = b.cpu()
    red = buf(1000, torch.float32)
    src = buf(1000, torch.float32)
    src.copy_(_inputs(rank, 1000, torch.float32, 13))
    comm.reduce(src, red, root=0)
    torch.cuda.synchronize()
    res["red"] = red.cpu()
    # ring exchange with send/recv (3 MiB + a ragged tail: several mailbox chunks)
    m = (3 << 20) // 4 + 3
    sb = torch.full((m,), float(rank), device="cuda")
    rb = torch.zeros(m, device="cuda")
    with group():
        comm.send(sb, (rank + 1) % n)
        comm.recv(rb, (rank - 1) % n)
    torch.cuda.synchronize()
    res["ring"] = rb[:: m // 7].cpu()
    assert comm.async_error() == 0
    comm.destroy()
    # plain numpy goes through the result queue (tensors would be shared by file descriptor and
    # vanish with this process); bf16 widens to fp32 exactly
    return {k: (v.float() if v.dtype == torch.bfloat16 else v).numpy() for k, v in res.items()}


def _check(results, n):
    import torch
    results = {r: {k: torch.from_numpy(v) for k, v in d.items()} for r, d in results.items()}
    for key in results[0]:
        if isinstance(key, tuple):
            _, dts, numel, op = key
            dtype = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.int32": torch.int32}[dts]
            ins = [_inputs(r, numel, dtype) for r in range(n)]
            acc_t = torch.float32 if dtype.is_floating_point else torch.int64
            acc = ins[0].to(acc_t)
            for x in ins[1:]:
                acc = acc + x.to(acc_t) if op == "sum" else torch.maximum(acc, x.to(acc_t))
            want = acc.to(dtype)
            for r in range(n):
                got = results[r][key]
                tol = 2 ** -6 if dtype == torch.bfloat16 else 1e-5
                assert torch.allclose(got.float(), want.float(), rtol=tol, atol=tol), (key, r)
    per = 4096 + 16
    ag = torch.cat([_inputs(r, per, torch.float32, 7) for r in range(n)])
    bigs = [_inputs(r, per * n, torch.float32, 9) for r in range(n)]
    tot = torch.stack(bigs).sum(0)
    for r in range(n):
        assert torch.equal(results[r]["ag"], ag)
        assert torch.allclose(results[r]["rs"], tot[r * per:(r + 1) * per], rtol=1e-5, atol=1e-5)
        want = torch.cat([bigs[p][r * per:(r + 1) * per] for p in range(n)])
        assert torch.equal(results[r]["a2a"], want)
        assert torch.equal(results[r]["bc"], _inputs(n - 1, 1000, torch.float32, 11))
        assert torch.equal(results[r]["ring"], torch.full_like(results[r]["ring"], float((r - 1) % n)))
    red = torch.stack([_inputs(r, 1000, torch.float32, 13) for r in range(n)]).sum(0)
    assert torch.allclose(results[0]["red"], red, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("registered", [True, False])
@pytest.mark.parametrize("algo", ["", "P2P", "NVLS"])
def test_collectives_all_gpus(registered, algo):
    n = min(_ngpus(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_colls_rank, n, args=(registered, algo), timeout=300)
    _check(res, n)


def test_two_gpus_when_more_exist():
    if _ngpus() < 4:
        pytest.skip("needs at least four GPUs")
    res = run_ranks(_colls_rank, 2, args=(True, ""), timeout=300)
    _check(res, 2)
