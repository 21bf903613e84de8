"""Expert-parallel dispatch / combine across real GPUs through the ncclEp* API."""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu


def _ep_rank(rank, nranks, uid, E, K, H, T, split=False):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    from nccl_b200.ops.ep import ExpertParallel
    comm = Communicator(nranks, rank, uid)
    ep = ExpertParallel(comm, E, T, H)
    res = {}
    for rep in range(3):
        g = torch.Generator().manual_seed(100 * rep + rank)
        x = torch.randn(T, H, generator=g).bfloat16().cuda()
        idx = torch.rand(T, E, generator=g).topk(K, dim=1).indices.to(torch.int64).cuda()
        w = torch.softmax(torch.randn(T, K, generator=g), dim=1).cuda()
        toks, scales, counts = ep.dispatch(x, idx, w, fp8=bool(rep % 2), send_only=split)
        if split:
            filler = torch.ones(1 << 20, device="cuda").mul_(2.0)   # work of the caller between the two halves
            ep.complete()
            del filler
        torch.cuda.synchronize()
        if rep % 2:
            y = (toks.view(torch.float8_e4m3fn).float().view(ep.El, ep.cap, H // 128, 128) * scales.unsqueeze(-1)).view(ep.El, ep.cap, H).bfloat16()
        else:
            y = toks
        # expert e multiplies by (e + 1)
        for el in range(ep.El):
            y[el] *= float(rank * ep.El + el + 1)
        out = ep.combine(y.contiguous(), send_only=split)
        if split:
            ep.complete()
        torch.cuda.synchronize()
        assert ep.mask() == [0] * nranks
        scale = torch.zeros(T, 1, device="cuda")
        for k in range(K):
            scale[:, 0] += w[:, k] * (idx[:, k] + 1).float()
        ref = x.float() * scale
        res["err%d" % rep] = float(((out.float() - ref).abs() / (ref.abs() + 1.0)).max())
        res["count%d" % rep] = int(counts.sum())
    assert comm.async_error() == 0
    ep.destroy()
    comm.destroy()
    return res


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("E,K,H,T", [(16, 2, 256, 32), (64, 8, 1024, 128)])
def test_ep_roundtrip(E, K, H, T, split):
    n = min(torch.cuda.device_count() if torch.cuda.is_available() else 0, 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    if E % n:
        pytest.skip("experts do not divide over the ranks")
    res = run_ranks(_ep_rank, n, args=(E, K, H, T, split), timeout=300)
    for rep in range(3):
        assert sum(res[r]["count%d" % rep] for r in range(n)) == n * T * K
        tol = 0.12 if rep % 2 else 0.03
        for r in range(n):
            assert res[r]["err%d" % rep] < tol, (rep, r, res[r])


def _ep_rank_layout(rank, nranks, uid, E, K, H, T, layout):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    from nccl_b200.ops.ep import ExpertParallel
    comm = Communicator(nranks, rank, uid)
    ep = ExpertParallel(comm, E, T, H, layout=layout)
    res = {}
    for rep in range(3):
        g = torch.Generator().manual_seed(100 * rep + rank)
        x = torch.randn(T, H, generator=g).bfloat16().cuda()
        idx = torch.rand(T, E, generator=g).topk(K, dim=1).indices.to(torch.int64).cuda()
        w = torch.softmax(torch.randn(T, K, generator=g), dim=1).cuda()
        toks, scales, counts = ep.dispatch(x, idx, w, fp8=False)
        torch.cuda.synchronize()
        ridx, rw = ep.recv_topk_idx, ep.recv_topk_weights
        # local experts (expert e multiplies by e + 1), pre-reduced with the weights that came with the token
        scale = (rw * (ridx + 1).clamp(min=0).float() * (ridx >= 0)).sum(-1, keepdim=True)
        y = (toks.float() * scale).bfloat16().contiguous()
        out = ep.combine(y)
        torch.cuda.synchronize()
        ref = x.float() * (w * (idx + 1).float()).sum(1, keepdim=True)
        res["err%d" % rep] = float(((out.float() - ref).abs() / (ref.abs() + 1.0)).max())
        res["count%d" % rep] = int(counts.sum())
        res["rows%d" % rep] = int((ridx >= 0).any(-1).sum())
        if layout == "flat":
            assert int(ep.recv_total[0]) == res["rows%d" % rep]
    assert comm.async_error() == 0
    ep.destroy()
    comm.destroy()
    return res


@pytest.mark.parametrize("layout", ["rank_major", "flat"])
def test_ep_layouts_with_one_copy_per_rank(layout):
    n = min(torch.cuda.device_count() if torch.cuda.is_available() else 0, 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    E, K, H, T = 8 * n, 4, 512, 64
    res = run_ranks(_ep_rank_layout, n, args=(E, K, H, T, layout), timeout=300)
    for rep in range(3):
        assert sum(res[r]["count%d" % rep] for r in range(n)) == n * T * K
        assert sum(res[r]["rows%d" % rep] for r in range(n)) <= n * T * min(K, n)
        for r in range(n):
            assert res[r]["err%d" % rep] < 0.03, (rep, r, res[r])


def _ep_rank_bindings_shape(rank, nranks, uid, E, K, H, T):
    """The same round trip written against the module with the reference bindings' call shapes."""
    import torch
    torch.cuda.set_device(rank)
    import nccl_b200.nccl4py.core as nccl
    import nccl_b200.nccl4py.ep as ep
    comm = nccl.Communicator.init(nranks, rank, nccl.UniqueId(uid))
    group = ep.Group.create(comm, ep.GroupConfig(num_experts=E, max_dispatch_tokens_per_rank=T, max_token_bytes=2 * H))
    El, cap = E // nranks, nranks * T
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator().manual_seed(rank)
    x = torch.randn(T, H, generator=g).bfloat16().cuda()
    idx = torch.rand(T, E, generator=g).topk(K, dim=1).indices.to(torch.int64).cuda()
    w = torch.softmax(torch.randn(T, K, generator=g), dim=1).cuda()
    toks = torch.empty(El, cap, H, dtype=torch.bfloat16, device="cuda")
    counts = torch.zeros(El, dtype=torch.int32, device="cuda")
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    handle = group.create_handle(ep.Layout.EXPERT_MAJOR, ep.Tensor(idx), stream=stream)
    handle.dispatch(ep.DispatchInputs(tokens=ep.Tensor(x), topk_weights=ep.Tensor(w)), ep.DispatchOutputs(tokens=ep.Tensor(toks)),
                    layout_info=ep.LayoutInfo(expert_counters=ep.Tensor(counts)), config=ep.DispatchConfig(), stream=stream)
    torch.cuda.synchronize()
    for el in range(El):
        toks[el] *= float(rank * El + el + 1)
    handle.combine(ep.CombineInputs(tokens=ep.Tensor(toks)), ep.CombineOutputs(tokens=ep.Tensor(out)), config=ep.CombineConfig(), stream=stream)
    torch.cuda.synchronize()
    ref = x.float() * (w * (idx + 1).float()).sum(1, keepdim=True)
    err = float(((out.float() - ref).abs() / (ref.abs() + 1.0)).max())
    total = int(counts.sum())
    handle.destroy()
    group.destroy()
    comm.destroy()
    return err, total


def test_ep_roundtrip_through_the_bindings_shaped_module():
    n = min(torch.cuda.device_count() if torch.cuda.is_available() else 0, 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    E, K, H, T = 8 * n, 4, 512, 64
    res = run_ranks(_ep_rank_bindings_shape, n, args=(E, K, H, T), timeout=300)
    assert sum(res[r][1] for r in range(n)) == n * T * K
    for r in range(n):
        assert res[r][0] < 0.03, res[r]
