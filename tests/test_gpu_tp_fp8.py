"""Block-scaled fp8 tcgen05 GEMM: quantisation kernels and the two-level accumulation against a
PyTorch fp32 reference of the same quantised operands; fused variants on several GPUs."""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu


def _dequant(q, s, block_rows):
    """q [R, K] e4m3, s [K/128, R/block_rows] -> fp32 [R, K]."""
    R, K = q.shape
    sc = s.t().contiguous()                                   # [R/block_rows, K/128]
    sc = sc.repeat_interleave(block_rows, 0).repeat_interleave(128, 1)
    return q.float() * sc


def _needs_sm100():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    if torch.cuda.get_device_capability()[0] < 10:
        pytest.skip("needs sm_100")


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (256, 512, 512), (1024, 768, 4096), (2048, 3584, 1024)])
def test_fp8_gemm_single_gpu(M, N, K):
    _needs_sm100()
    from nccl_b200 import Communicator, get_unique_id
    from nccl_b200.ops.tp import TensorParallel
    torch.cuda.set_device(0)
    comm = Communicator(1, 0, get_unique_id())
    tp = TensorParallel(comm, 4096, 4096)
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = (torch.randn(M, K, device="cuda", generator=g) * torch.rand(M, 1, device="cuda", generator=g) * 4).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    xq, xs = tp.quantize_fp8(x, 1)
    wq, ws = tp.quantize_fp8(w, 128)
    torch.cuda.synchronize()
    # quantisation: scales are amax / 448 per block and the round trip is within e4m3 precision
    xd, wd = _dequant(xq, xs, 1), _dequant(wq, ws, 128)
    amax = x.float().view(M, K // 128, 128).abs().amax(-1)
    torch.testing.assert_close(xs.t().contiguous(), (amax.clamp_min(1e-10) / 448), rtol=1e-5, atol=1e-12)
    assert (xd - x.float()).abs().max() <= 0.07 * x.float().abs().max()
    assert (wd - w.float()).abs().max() <= 0.07 * w.float().abs().max()
    ref = xd @ wd.t()
    for _ in range(2):
        y = tp.gemm_fp8(xq, xs, wq, ws)
        torch.cuda.synchronize()
        err = (y.float() - ref).abs().max().item()
        scale = ref.abs().max().item()
        assert err <= 1e-2 * scale + 1e-2, (err, scale)
    assert comm.async_error() == 0
    tp.destroy()
    comm.destroy()


def _rank(rank, nranks, uid, M, N, K):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    from nccl_b200.ops.tp import TensorParallel
    comm = Communicator(nranks, rank, uid)
    tp = TensorParallel(comm, M, max(N, 256))
    n = nranks
    gx = torch.Generator().manual_seed(5)
    x_full = torch.randn(M, K, generator=gx).bfloat16()
    w_full = (torch.randn(N, K, generator=gx) * 0.05).bfloat16()
    out = {}
    # row-parallel: K is sharded; every rank quantises its slice
    ks = K // n
    xs_, ws_ = x_full[:, rank * ks:(rank + 1) * ks].contiguous().cuda(), w_full[:, rank * ks:(rank + 1) * ks].contiguous().cuda()
    xq, xsc = tp.quantize_fp8(xs_, 1)
    wq, wsc = tp.quantize_fp8(ws_, 128)
    for _ in range(2):
        y = tp.gemm_reduce_scatter_fp8(xq, xsc, wq, wsc)
        torch.cuda.synchronize()
    out["rs"] = y.float().cpu().numpy()
    out["rs_q"] = (xq.float().cpu().numpy(), xsc.cpu().numpy(), wq.float().cpu().numpy(), wsc.cpu().numpy())
    # column-parallel: rows of x are sharded; each rank quantises its rows into the shared window
    gq, gs = tp.alloc_gathered_fp8(M, K)
    rows = M // n
    wq2, wsc2 = tp.quantize_fp8(w_full.cuda(), 128)
    for _ in range(2):
        gq.view(torch.uint8).zero_()
        gs.zero_()
        mine_q, mine_s = tp.quantize_fp8(x_full[rank * rows:(rank + 1) * rows].contiguous().cuda(), 1)
        gq[rank * rows:(rank + 1) * rows].view(torch.uint8).copy_(mine_q.view(torch.uint8))
        gs[:, rank * rows:(rank + 1) * rows].copy_(mine_s)
        torch.cuda.synchronize()
        y2 = tp.all_gather_gemm_fp8(gq, wq2, wsc2)
        torch.cuda.synchronize()
    out["ag"] = y2.float().cpu().numpy()
    out["ag_q"] = (gq.float().cpu().numpy(), gs.cpu().numpy(), wq2.float().cpu().numpy(), wsc2.cpu().numpy())
    assert comm.async_error() == 0
    tp.destroy()
    comm.destroy()
    return out


@pytest.mark.parametrize("M,N,K", [(1024, 512, 1024), (2048, 1024, 2048)])
def test_fp8_fused_multi_gpu(M, N, K):
    _needs_sm100()
    n = min(torch.cuda.device_count(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_rank, n, args=(M, N, K), timeout=300)
    rows = M // n

    def deq(q, s, br):
        return _dequant(torch.from_numpy(q), torch.from_numpy(s), br)

    ref_rs = sum(deq(res[r]["rs_q"][0], res[r]["rs_q"][1], 1) @ deq(res[r]["rs_q"][2], res[r]["rs_q"][3], 128).t() for r in range(n))
    scale = ref_rs.abs().max().item()
    for r in range(n):
        rs = torch.from_numpy(res[r]["rs"])
        assert (rs - ref_rs[r * rows:(r + 1) * rows]).abs().max().item() <= 2e-2 * scale + 2e-2
        q = res[r]["ag_q"]
        ref_ag = deq(q[0], q[1], 1) @ deq(q[2], q[3], 128).t()
        ag = torch.from_numpy(res[r]["ag"])
        assert (ag - ref_ag).abs().max().item() <= 1e-2 * ref_ag.abs().max().item() + 1e-2
        # the gathered operand is complete and identical on every rank
        assert (torch.from_numpy(q[0]) == torch.from_numpy(res[0]["ag_q"][0])).all()
