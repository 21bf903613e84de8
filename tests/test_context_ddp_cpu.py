"""Data-parallel gradient buckets, ring attention and the Ulysses all-to-all swap on CPU ranks
(host-only communicators over sockets), each checked against a single-process PyTorch reference."""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

ENV = {"NCCL_B200_HOST_ONLY": "1", "NCCL_SOCKET_IFNAME": "lo"}


def _model():
    torch.manual_seed(3)
    return torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.Tanh(), torch.nn.Linear(40, 17), torch.nn.Tanh(), torch.nn.Linear(17, 5))


def _data(rank):
    g = torch.Generator().manual_seed(100 + rank)
    return torch.randn(6, 24, generator=g), torch.randn(6, 5, generator=g)


def _ddp_rank(rank, nranks, uid):
    import torch
    torch.set_num_threads(2)
    from nccl_b200 import Communicator
    from nccl_b200.parallel.ddp import GradientBuckets
    comm = Communicator(nranks, rank, uid)
    model = _model()
    buckets = GradientBuckets(comm, list(model.parameters()), bucket_bytes=2048)   # several small buckets
    out = []
    for _ in range(2):
        buckets.zero_grad()
        x, y = _data(rank)
        ((model(x) - y) ** 2).mean().backward()
        buckets.finish()
        out.append([p.grad.clone().numpy() for p in model.parameters()])
    nb, launched = len(buckets.buckets), buckets.launched
    buckets.close()
    comm.destroy()
    return out, nb, launched


def test_gradient_buckets_average():
    import numpy as np
    n = 3
    res = run_ranks(_ddp_rank, n, env=ENV, timeout=200)
    model = _model()
    ref = [torch.zeros_like(p) for p in model.parameters()]
    for r in range(n):
        model.zero_grad()
        x, y = _data(r)
        ((model(x) - y) ** 2).mean().backward()
        for a, p in zip(ref, model.parameters()):
            a += p.grad / n
    for r in range(n):
        grads, nb, launched = res[r]
        assert nb >= 3 and launched == 2 * nb
        for step in range(2):
            for g, a in zip(grads[step], ref):
                np.testing.assert_allclose(g, a.numpy(), rtol=1e-5, atol=1e-6)


def _qkv(B, H, S_all, D):
    g = torch.Generator().manual_seed(11)
    return [torch.randn(B, H, S_all, D, generator=g) for _ in range(3)]


def _ring_rank(rank, nranks, uid, causal):
    import torch
    torch.set_num_threads(2)
    from nccl_b200 import Communicator
    from nccl_b200.parallel.context import ring_attention, ulysses_attention
    comm = Communicator(nranks, rank, uid)
    B, H, S_all, D = 2, 6, 8 * nranks, 16
    q, k, v = _qkv(B, H, S_all, D)
    S = S_all // nranks
    sl = slice(rank * S, (rank + 1) * S)
    ring = ring_attention(comm, q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous(), causal=causal)
    # Ulysses layout is [batch, local sequence, heads, dim]
    to_bshd = lambda t: t[:, :, sl].transpose(1, 2).contiguous()   # noqa: E731
    uly = ulysses_attention(comm, to_bshd(q), to_bshd(k), to_bshd(v), causal=causal).transpose(1, 2)
    comm.destroy()
    return ring.numpy(), uly.numpy()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("n", [2, 3])
def test_ring_and_ulysses_attention(n, causal):
    import numpy as np
    res = run_ranks(_ring_rank, n, args=(causal,), env=ENV, timeout=200)
    B, H, S_all, D = 2, 6, 8 * n, 16
    q, k, v = _qkv(B, H, S_all, D)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal).numpy()
    S = S_all // n
    for r in range(n):
        np.testing.assert_allclose(res[r][0], ref[:, :, r * S:(r + 1) * S], rtol=2e-4, atol=2e-5)
        np.testing.assert_allclose(res[r][1], ref[:, :, r * S:(r + 1) * S], rtol=2e-4, atol=2e-5)


def test_example_script_runs_on_cpu_ranks():
    """examples/train_ddp_ring_attention.py under torch.distributed.run with two CPU ranks."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_B200_HOST_ONLY="1", NCCL_SOCKET_IFNAME="lo", OMP_NUM_THREADS="2")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29631", os.path.join(root, "examples", "train_ddp_ring_attention.py")],
                       env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert p.stdout.count("ring attention max error") == 2
