"""Device API: device communicators, LSA barriers, low-latency sessions and the fused
all-reduce + residual + RMSNorm kernel, one process per GPU (one rank when a single GPU is present).
"""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu


def _ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _rank(rank, nranks, uid):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    from nccl_b200.ops.devapi import DeviceComm, query_properties
    comm = Communicator(nranks, rank, uid)
    props = query_properties(comm)
    assert props["deviceApiSupport"] == 1 and props["nRanks"] == nranks
    dc = DeviceComm(comm, barriers=64, ll_blocks=2, ll_slots=128, gin_signals=2, gin_counters=1)
    res = {"multimem": props["multimemSupport"]}
    # all-reduce written with the device headers
    for dtype, numel in ((torch.float32, 1 << 18), (torch.bfloat16, (1 << 16) + 8)):
        x = dc.symmetric(numel, dtype)
        y = dc.symmetric(numel, dtype)
        g = torch.Generator().manual_seed(11 + rank)
        x.copy_(torch.randn(numel, generator=g).to(dtype))
        modes = [False] + ([True] if props["multimemSupport"] and nranks > 1 else [])
        for mm in modes:
            y.zero_()
            torch.cuda.synchronize()
            for _ in range(3):   # repeated launches exercise the persistent barrier epochs
                dc.all_reduce(x, y, multimem=mm)
            assert dc.status() == 0
            res[("ar", str(dtype), mm)] = y.float().cpu().numpy()
    # fused all-reduce + residual + RMSNorm
    T, H = 37, 4096
    part = dc.symmetric(T * H, torch.bfloat16).view(T, H)
    resid = dc.symmetric(T * H, torch.bfloat16).view(T, H)
    out = dc.symmetric(T * H, torch.bfloat16).view(T, H)
    w = (torch.randn(H, generator=torch.Generator().manual_seed(5)) * 0.1 + 1).to(torch.bfloat16).cuda()
    modes = [0, 2] + ([1] if props["multimemSupport"] and nranks > 1 else [])
    for mode in modes:
        part.copy_(torch.randn(T, H, generator=torch.Generator().manual_seed(21 + rank)).to(torch.bfloat16))
        resid.copy_(torch.randn(T, H, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16))
        out.zero_()
        torch.cuda.synchronize()
        comm.all_reduce(torch.zeros(8, device="cuda"))   # every rank has written its inputs
        torch.cuda.synchronize()
        dc.ar_rmsnorm(part, resid, out, w, eps=1e-5, mode=mode)
        assert dc.status() == 0
        res[("norm", mode)] = (out.float().cpu().numpy(), resid.float().cpu().numpy())
    # low-latency session
    vals = torch.randn(2, 128, 2, generator=torch.Generator().manual_seed(40 + rank)).cuda()
    o = torch.zeros_like(vals)
    for _ in range(3):
        dc.ll_sum(vals, o, ctas=2)
    assert dc.status() == 0
    res["ll"] = o.cpu().numpy()
    # one-sided put + signal around the ring
    both = dc.symmetric(2 * 1000, torch.float32)
    snd, rcv = both[:1000], both[1000:]
    for it in range(3):
        snd.fill_(100.0 * it + rank)
        torch.cuda.synchronize()
        comm.all_reduce(torch.zeros(8, device="cuda"))   # nobody overwrites a receive region that is still being read
        torch.cuda.synchronize()
        dc.gin_ring(snd, rcv)
        assert dc.status() == 0
        assert float(rcv[0]) == 100.0 * it + (rank - 1) % nranks and float(rcv[-1]) == float(rcv[0])
    dc.destroy()
    comm.destroy()
    return res


def _check(results, n):
    import numpy as np
    for dtype, numel in ((torch.float32, 1 << 18), (torch.bfloat16, (1 << 16) + 8)):
        xs = [torch.randn(numel, generator=torch.Generator().manual_seed(11 + r)).to(dtype).float() for r in range(n)]
        ref = sum(xs).numpy()
        for r in range(n):
            for mm in (False, True):
                k = ("ar", str(dtype), mm)
                if k in results[r]:
                    tol = 1e-5 if dtype == torch.float32 else 3e-2
                    np.testing.assert_allclose(results[r][k], ref, rtol=tol, atol=tol * 4)
    T, H = 37, 4096
    parts = [torch.randn(T, H, generator=torch.Generator().manual_seed(21 + r)).to(torch.bfloat16).float() for r in range(n)]
    resid = torch.randn(T, H, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).float()
    w = (torch.randn(H, generator=torch.Generator().manual_seed(5)) * 0.1 + 1).to(torch.bfloat16).float()
    x = (sum(parts) + resid).to(torch.bfloat16).float()
    ref = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w
    for r in range(n):
        for mode in (0, 1, 2):
            if ("norm", mode) in results[r]:
                o, rs = results[r][("norm", mode)]
                np.testing.assert_allclose(rs, x.numpy(), rtol=2e-2, atol=2e-2)
                np.testing.assert_allclose(o, ref.numpy(), rtol=3e-2, atol=3e-2)
    ll = sum(torch.randn(2, 128, 2, generator=torch.Generator().manual_seed(40 + r)) for r in range(n)).numpy()
    for r in range(n):
        np.testing.assert_allclose(results[r]["ll"], ll, rtol=1e-5, atol=1e-5)


def test_device_api_one_rank():
    if _ngpus() < 1:
        pytest.skip("needs a GPU")
    _check(run_ranks(_rank, 1), 1)


@pytest.mark.parametrize("n", [2, 4, 8])
def test_device_api_multi(n):
    if _ngpus() < n:
        pytest.skip(f"needs {n} GPUs")
    _check(run_ranks(_rank, n), n)


def _rank_gin_proxy(rank, nranks, uid):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    from nccl_b200.ops.devapi import DeviceComm, query_properties
    comm = Communicator(nranks, rank, uid)
    assert query_properties(comm)["ginType"] == 2   # served by a host proxy thread
    dc = DeviceComm(comm, barriers=4, gin_signals=2, gin_counters=1)
    both = dc.symmetric(2 * 4096, torch.float32)
    snd, rcv = both[:4096], both[4096:]
    seen = []
    for it in range(5):
        snd.fill_(100.0 * it + rank)
        torch.cuda.synchronize()
        comm.all_reduce(torch.zeros(8, device="cuda"))
        torch.cuda.synchronize()
        dc.gin_ring(snd, rcv)
        torch.cuda.synchronize()
        assert dc.status() == 0
        seen.append((float(rcv[0]), float(rcv[-1])))
    dc.destroy()
    comm.destroy()
    return seen


@pytest.mark.parametrize("n", [1, 2])
def test_put_and_signal_through_the_host_proxy(n):
    """NCCL_GIN_TYPE=PROXY: the kernel only queues descriptors; a host thread runs the copies on the copy engines
    and the signal / counter updates behind them. Same ring exchange as with peer stores, same result."""
    if _ngpus() < n:
        pytest.skip(f"needs {n} GPUs")
    res = run_ranks(_rank_gin_proxy, n, env={"NCCL_GIN_TYPE": "PROXY"})
    for r in range(n):
        assert res[r] == [(100.0 * it + (r - 1) % n,) * 2 for it in range(5)], (r, res[r])
