"""FSDP engine, fused AdamW kernel and pipeline stages on GPUs (one process per GPU)."""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu


def _ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def test_fused_adamw_matches_formula():
    if _ngpus() < 1:
        pytest.skip("needs a GPU")
    import ctypes
    from nccl_b200 import _lib
    lib = _lib.load()
    lib.b200FusedAdamW.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_size_t] + [ctypes.c_float] * 6 + [ctypes.c_int, ctypes.c_void_p]
    n = (1 << 20) + 8 + 3
    g = torch.Generator().manual_seed(0)
    w = torch.randn(n, generator=g).cuda()
    m = (torch.randn(n, generator=g) * 0.1).cuda()
    v = (torch.rand(n, generator=g) * 0.01).cuda()
    grad = torch.randn(n, generator=g).to(torch.bfloat16).cuda()
    p = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    lr, b1, b2, eps, wd, scale, step = 1e-2, 0.9, 0.95, 1e-8, 0.1, 0.5, 3
    gw = grad.float() * scale
    m_ref = b1 * m + (1 - b1) * gw
    v_ref = b2 * v + (1 - b2) * gw * gw
    w_ref = w * (1 - lr * wd) - lr * (m_ref / (1 - b1 ** step)) / (v_ref.sqrt() / (1 - b2 ** step) ** 0.5 + eps)
    rc = lib.b200FusedAdamW(w.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(), p.data_ptr(), n, lr, b1, b2, eps, wd, scale, step,
                            torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    torch.testing.assert_close(m, m_ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(v, v_ref, rtol=1e-5, atol=1e-7)
    torch.testing.assert_close(w, w_ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(p.float(), w_ref.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-2)


def _fsdp_rank(rank, nranks, uid):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    from nccl_b200.models import llama as M
    from nccl_b200.parallel.fsdp import FSDPEngine
    comm = Communicator(nranks, rank, uid)
    cfg = M.LlamaConfig(layers=3, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=1024, rope_theta=10000.0)
    lr = 1e-2
    eng = FSDPEngine(comm, cfg, device="cuda", seed=1, lr=lr, weight_decay=0.0)
    data = []
    for r in range(nranks):
        g = torch.Generator().manual_seed(50 + r)
        data.append((torch.randint(0, cfg.vocab, (2, 64), generator=g), torch.randint(0, cfg.vocab, (2, 64), generator=g)))
    tok, tgt = data[rank][0].pin_memory(), data[rank][1].pin_memory()
    losses = [float(eng.step(tok, tgt)) for _ in range(2)]
    got = eng.full_params()
    colls = eng.collectives
    eng.close()
    comm.destroy()
    # plain autograd + the same AdamW on whole buffers
    gen = torch.Generator().manual_seed(1)
    master = [M.init_flat(s, gen).float().cuda() for _, s in M.unit_specs(cfg)]
    m = [torch.zeros_like(f) for f in master]
    v = [torch.zeros_like(f) for f in master]
    b1, b2, eps = 0.9, 0.95, 1e-8
    ref_losses = []
    for step in (1, 2):
        ps = [f.to(torch.bfloat16).requires_grad_(True) for f in master]
        grads = [torch.zeros_like(f) for f in master]
        for r in range(nranks):
            loss = M.reference_loss(ps, cfg, data[r][0].cuda(), data[r][1].cuda())
            if r == rank:
                ref_losses.append(float(loss.detach()))
            for a, b in zip(grads, torch.autograd.grad(loss, ps)):
                a += b.float()
        for i in range(len(master)):
            gq = grads[i].to(torch.bfloat16).float() / nranks
            m[i] = b1 * m[i] + (1 - b1) * gq
            v[i] = b2 * v[i] + (1 - b2) * gq * gq
            master[i] = master[i] - lr * (m[i] / (1 - b1 ** step)) / (v[i].sqrt() / (1 - b2 ** step) ** 0.5 + eps)
    bad = [float(((got[i].cuda() - master[i].to(torch.bfloat16).float()).abs() > 0.5 * lr).float().mean()) for i in range(len(master))]
    return losses, ref_losses, bad, colls


@pytest.mark.parametrize("n", [1, 2, 4, 8])
def test_fsdp_step_matches_autograd(n):
    if _ngpus() < n:
        pytest.skip(f"needs {n} GPUs")
    res = run_ranks(_fsdp_rank, n, timeout=300)
    for r in range(n):
        losses, ref, bad, colls = res[r]
        for a, b in zip(losses, ref):
            assert abs(a - b) < 3e-2 * max(1.0, abs(b)), (losses, ref)
        assert max(bad) < 0.03, bad
        assert colls >= 2 * 3 * 5   # two steps x (2 gathers + 1 reduce-scatter) x 5 units, roughly


def _pipe_rank(rank, nranks, uid):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    from nccl_b200.models import llama as M
    from nccl_b200.parallel.pipeline import PipelineStage
    comm = Communicator(nranks, rank, uid)
    cfg = M.LlamaConfig(layers=4, hidden=256, heads=4, kv_heads=2, ffn=512, vocab=1024, rope_theta=10000.0)
    st = PipelineStage(comm, cfg, device="cuda", seed=3)
    g = torch.Generator().manual_seed(9)
    toks = [torch.randint(0, cfg.vocab, (1, 64), generator=g) for _ in range(3)]
    tgts = [torch.randint(0, cfg.vocab, (1, 64), generator=g) for _ in range(3)]
    loss = st.forward_backward(toks, tgts)
    torch.cuda.synchronize()
    out = None if loss is None else float(loss)
    gen = torch.Generator().manual_seed(3)
    ps = [M.init_flat(s, gen).cuda().requires_grad_(True) for _, s in M.unit_specs(cfg)]
    total = sum(M.reference_loss(ps, cfg, a.cuda(), b.cuda()) for a, b in zip(toks, tgts)) / 3
    total.backward()
    err = {i: float((p.grad.float() - ps[i].grad.float()).abs().max() / (ps[i].grad.float().abs().max() + 1e-6)) for i, p in st.params.items()}
    comm.destroy()
    return out, float(total.detach()), err


@pytest.mark.parametrize("n", [2, 4])
def test_pipeline_matches_autograd(n):
    if _ngpus() < n:
        pytest.skip(f"needs {n} GPUs")
    res = run_ranks(_pipe_rank, n, timeout=300)
    assert abs(res[n - 1][0] - res[n - 1][1]) < 3e-2 * max(1.0, abs(res[n - 1][1]))
    for r in range(n):
        assert max(res[r][2].values()) < 0.1, res[r][2]


def _ddp_ctx_rank(rank, nranks, uid):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    from nccl_b200.parallel.context import ring_attention, ulysses_attention
    from nccl_b200.parallel.ddp import GradientBuckets
    comm = Communicator(nranks, rank, uid)
    torch.manual_seed(3)
    model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 128)).cuda()
    buckets = GradientBuckets(comm, list(model.parameters()), bucket_bytes=256 << 10)
    g = torch.Generator().manual_seed(100 + rank)
    x, y = torch.randn(32, 256, generator=g).cuda(), torch.randn(32, 128, generator=g).cuda()
    for _ in range(2):
        buckets.zero_grad()
        ((model(x) - y) ** 2).mean().backward()
        buckets.finish()
    torch.cuda.synchronize()
    grads = [p.grad.float().cpu().numpy().copy() for p in model.parameters()]
    nb = len(buckets.buckets)
    buckets.close()
    # sequence-parallel attention on the same communicator
    B, H, S_all, D = 2, 8, 64 * nranks, 32
    gq = torch.Generator().manual_seed(11)
    q, k, v = [torch.randn(B, H, S_all, D, generator=gq) for _ in range(3)]
    S = S_all // nranks
    sl = slice(rank * S, (rank + 1) * S)
    loc = [t[:, :, sl].contiguous().cuda() for t in (q, k, v)]
    ring = ring_attention(comm, *loc, causal=True)
    uly = ulysses_attention(comm, *[t.transpose(1, 2).contiguous() for t in loc], causal=True).transpose(1, 2)
    torch.cuda.synchronize()
    assert comm.async_error() == 0
    out = grads, nb, ring.cpu().numpy(), uly.cpu().numpy()
    comm.destroy()
    return out


@pytest.mark.parametrize("n", [2, 4])
def test_gradient_buckets_and_context_parallel(n):
    import numpy as np
    if _ngpus() < n:
        pytest.skip("needs %d GPUs" % n)
    res = run_ranks(_ddp_ctx_rank, n, timeout=300)
    torch.manual_seed(3)
    model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 128))
    ref = [torch.zeros_like(p) for p in model.parameters()]
    for r in range(n):
        model.zero_grad()
        g = torch.Generator().manual_seed(100 + r)
        x, y = torch.randn(32, 256, generator=g), torch.randn(32, 128, generator=g)
        ((model(x) - y) ** 2).mean().backward()
        for a, p in zip(ref, model.parameters()):
            a += p.grad / n
    B, H, S_all, D = 2, 8, 64 * n, 32
    gq = torch.Generator().manual_seed(11)
    q, k, v = [torch.randn(B, H, S_all, D, generator=gq) for _ in range(3)]
    att = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True).numpy()
    S = S_all // n
    for r in range(n):
        grads, nb, ring, uly = res[r]
        assert nb >= 2
        for gg, a in zip(grads, ref):
            np.testing.assert_allclose(gg, a.numpy(), rtol=2e-3, atol=2e-5)
        np.testing.assert_allclose(ring, att[:, :, r * S:(r + 1) * S], rtol=2e-3, atol=2e-4)
        np.testing.assert_allclose(uly, att[:, :, r * S:(r + 1) * S], rtol=2e-3, atol=2e-4)
