"""tcgen05 GEMM kernels: plain on one GPU, fused with reduce-scatter / all-gather on several."""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu


def _ref(x, w):
    return (x.float() @ w.float().t())


def _gemm_rank(rank, nranks, uid, M, N, K):
    import torch
    from nccl_b200 import Communicator
    from nccl_b200.ops.tp import TensorParallel
    torch.cuda.set_device(0)
    comm = Communicator(1, 0, uid)
    tp = TensorParallel(comm, 4096, 4096)
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
    for _ in range(2):
        y = tp.gemm(x, w)
        torch.cuda.synchronize()
        ref = _ref(x, w)
        err = (y.float() - ref).abs().max().item()
        scale = ref.abs().max().item()
        assert err <= 1e-2 * scale + 1e-2, (err, scale)
    assert comm.async_error() == 0
    tp.destroy()
    comm.destroy()
    return True


# pair = 1: two CTAs per 256 x 256 tile (tcgen05 cta_group::2) where the row count allows; 0: one CTA per 128 x 256 tile
@pytest.mark.parametrize("pair", [1, 0])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1024, 768, 4096), (2048, 3584, 1024), (4096, 4096, 512)])
def test_gemm_single_gpu(M, N, K, pair):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    if torch.cuda.get_device_capability()[0] < 10:
        pytest.skip("needs sm_100")
    if pair == 0 and (M, N, K) not in ((256, 512, 256), (2048, 3584, 1024)):
        pytest.skip("shape covered with the default kernel choice")
    assert run_ranks(_gemm_rank, 1, args=(M, N, K), env={"NCCL_B200_TP_PAIR": str(pair)}, timeout=200)[0] is True


def _tp_rank(rank, nranks, uid, M, N, K):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    from nccl_b200.ops.tp import TensorParallel
    comm = Communicator(nranks, rank, uid)
    tp = TensorParallel(comm, M, max(N, 256))
    n = nranks
    out = {}
    # row-parallel: every rank holds a K-slice of x and w; the product is summed and row-scattered
    gx = torch.Generator().manual_seed(5)
    x_full = torch.randn(M, K, generator=gx).bfloat16()
    w_full = (torch.randn(N, K, generator=gx) * 0.05).bfloat16()
    ks = K // n
    xs = x_full[:, rank * ks:(rank + 1) * ks].contiguous().cuda()
    ws = w_full[:, rank * ks:(rank + 1) * ks].contiguous().cuda()
    for _ in range(2):
        y = tp.gemm_reduce_scatter(xs, ws)
        torch.cuda.synchronize()
    out["rs"] = y.float().cpu().numpy()
    # column-parallel: rows of x are sharded; weights w_col [N, K] local
    xg = tp.alloc_gathered(M, K)
    rows = M // n
    for rep in range(2):
        xg.zero_()
        xg[rank * rows:(rank + 1) * rows].copy_(x_full[rank * rows:(rank + 1) * rows].cuda())
        torch.cuda.synchronize()
        y2 = tp.all_gather_gemm(xg, w_full.cuda())
        torch.cuda.synchronize()
    out["ag"] = y2.float().cpu().numpy()
    out["xg"] = xg.float().cpu().numpy()
    assert comm.async_error() == 0
    tp.destroy()
    comm.destroy()
    return out


@pytest.mark.parametrize("pair", [1, 0])
@pytest.mark.parametrize("M,N,K", [(1024, 512, 1024), (2048, 1024, 2048)])
def test_fused_tp_multi_gpu(M, N, K, pair):
    n = min(torch.cuda.device_count() if torch.cuda.is_available() else 0, 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    if torch.cuda.get_device_capability()[0] < 10:
        pytest.skip("needs sm_100")
    res = run_ranks(_tp_rank, n, args=(M, N, K), env={"NCCL_B200_TP_PAIR": str(pair)}, timeout=300)
    gx = torch.Generator().manual_seed(5)
    x_full = torch.randn(M, K, generator=gx).bfloat16()
    w_full = (torch.randn(N, K, generator=gx) * 0.05).bfloat16()
    ref = _ref(x_full, w_full)
    scale = ref.abs().max().item()
    rows = M // n
    for r in range(n):
        rs = torch.from_numpy(res[r]["rs"])
        assert (rs - ref[r * rows:(r + 1) * rows]).abs().max().item() <= 2e-2 * scale + 2e-2
        assert torch.equal(torch.from_numpy(res[r]["xg"]), x_full.float())
        ag = torch.from_numpy(res[r]["ag"])
        assert (ag - ref).abs().max().item() <= 1e-2 * scale + 1e-2
