"""FSDP / ZeRO-3 engine and pipeline stages on CPU ranks (host-only communicators over sockets),
checked against plain single-process autograd on the same random-init model."""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

ENV = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}


def _fsdp_rank(rank, nranks, uid):
    import torch
    torch.manual_seed(0)
    torch.set_num_threads(2)
    from nccl_b200 import Communicator
    from nccl_b200.models.llama import LlamaConfig
    from nccl_b200.parallel.fsdp import FSDPEngine
    comm = Communicator(nranks, rank, uid)
    cfg = LlamaConfig.tiny(layers=3)
    eng = FSDPEngine(comm, cfg, device="cpu", seed=1, lr=1e-2, weight_decay=0.0)
    g = torch.Generator().manual_seed(50 + rank)
    tok = torch.randint(0, cfg.vocab, (2, 16), generator=g)
    tgt = torch.randint(0, cfg.vocab, (2, 16), generator=g)
    losses = [float(eng.step(tok, tgt)) for _ in range(2)]
    params = [p.numpy() for p in eng.full_params()]
    comm.destroy()
    return losses, params


def test_fsdp_matches_autograd():
    import numpy as np
    from nccl_b200.models import llama as M
    n = 2
    res = run_ranks(_fsdp_rank, n, env=ENV, timeout=300)
    cfg = M.LlamaConfig.tiny(layers=3)
    gen = torch.Generator().manual_seed(1)
    flats = [M.init_flat(s, gen) for _, s in M.unit_specs(cfg)]
    master = [f.float() for f in flats]
    m = [torch.zeros_like(f) for f in master]
    v = [torch.zeros_like(f) for f in master]
    data = []
    for r in range(n):
        g = torch.Generator().manual_seed(50 + r)
        data.append((torch.randint(0, cfg.vocab, (2, 16), generator=g), torch.randint(0, cfg.vocab, (2, 16), generator=g)))
    lr, b1, b2, eps = 1e-2, 0.9, 0.95, 1e-8
    for step in (1, 2):
        ps = [f.to(torch.bfloat16).requires_grad_(True) for f in master]
        ref_losses = []
        grads = [torch.zeros_like(f) for f in master]
        for r in range(n):
            loss = M.reference_loss(ps, cfg, *data[r])
            gs = torch.autograd.grad(loss, ps)
            ref_losses.append(float(loss))
            for a, b in zip(grads, gs):
                a += b.float()   # the library reduces bf16 gradients with fp32 accumulation
        for r in range(n):
            assert abs(res[r][0][step - 1] - ref_losses[r]) < 2e-2 * max(1.0, abs(ref_losses[r]))
        for i in range(len(master)):
            gq = grads[i].to(torch.bfloat16).float() / n
            m[i] = b1 * m[i] + (1 - b1) * gq
            v[i] = b2 * v[i] + (1 - b2) * gq * gq
            master[i] = master[i] - lr * (m[i] / (1 - b1 ** step)) / (v[i].sqrt() / (1 - b2 ** step) ** 0.5 + eps)
    for r in range(n):
        for i in range(len(master)):
            got = res[r][1][i]
            want = master[i].to(torch.bfloat16).float().numpy()
            # Adam's first steps move every weight by about lr; allow a fraction of that for sign flips of tiny gradients
            assert np.mean(np.abs(got - want) > 0.5 * lr) < 0.02, "unit %d differs" % i


def _pipe_rank(rank, nranks, uid):
    import torch
    torch.set_num_threads(2)
    from nccl_b200 import Communicator
    from nccl_b200.models.llama import LlamaConfig
    from nccl_b200.parallel.pipeline import PipelineStage
    comm = Communicator(nranks, rank, uid)
    cfg = LlamaConfig.tiny(layers=4)
    st = PipelineStage(comm, cfg, device="cpu", seed=3)
    g = torch.Generator().manual_seed(9)
    toks = [torch.randint(0, cfg.vocab, (1, 16), generator=g) for _ in range(3)]
    tgts = [torch.randint(0, cfg.vocab, (1, 16), generator=g) for _ in range(3)]
    loss = st.forward_backward(toks, tgts)
    grads = {i: p.grad.float().numpy() for i, p in st.params.items()}
    comm.destroy()
    return (None if loss is None else float(loss)), grads


def test_pipeline_matches_autograd():
    import numpy as np
    from nccl_b200.models import llama as M
    n = 2
    res = run_ranks(_pipe_rank, n, env=ENV, timeout=300)
    cfg = M.LlamaConfig.tiny(layers=4)
    gen = torch.Generator().manual_seed(3)
    ps = [M.init_flat(s, gen).requires_grad_(True) for _, s in M.unit_specs(cfg)]
    g = torch.Generator().manual_seed(9)
    toks = [torch.randint(0, cfg.vocab, (1, 16), generator=g) for _ in range(3)]
    tgts = [torch.randint(0, cfg.vocab, (1, 16), generator=g) for _ in range(3)]
    total = sum(M.reference_loss(ps, cfg, a, b) for a, b in zip(toks, tgts)) / 3
    total.backward()
    assert abs(res[n - 1][0] - float(total)) < 2e-2 * max(1.0, abs(float(total)))
    for r in range(n):
        for i, got in res[r][1].items():
            want = ps[i].grad.float().numpy()
            scale = np.abs(want).max() + 1e-6
            assert np.abs(got - want).max() < 0.08 * scale, "unit %d on stage %d" % (i, r)
