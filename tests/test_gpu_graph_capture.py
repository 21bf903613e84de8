"""Collectives captured into a CUDA graph and replayed with changing inputs.

Everything a kernel needs across launches (barrier epochs, flagged-line epochs, mailbox sequence
numbers) lives in device memory, so a captured sequence can be replayed any number of times: an
all-reduce, an all-gather, a group of small all-reduces (one aggregated launch) and a grouped
send / receive pair are captured once and replayed ten times, each time over new input values,
and compared with plain PyTorch arithmetic. Runs on one GPU (one-rank communicator) and on two.
"""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402
from test_gpu_multi import _ngpus, _sym_tensor  # noqa: E402

pytestmark = pytest.mark.gpu


def _capture_rank(rank, nranks, uid, registered):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator, group
    comm = Communicator(nranks, rank, uid)
    n = nranks
    numel = 4096

    def buf(k):
        return _sym_tensor(comm, k, torch.float32) if registered and n > 1 else torch.zeros(k, device="cuda")

    x, y = buf(numel), buf(numel)
    g_in, g_out = buf(numel), buf(numel * n)
    small_in = [buf(64 + 8 * i) for i in range(6)]
    small_out = [buf(64 + 8 * i) for i in range(6)]
    sb, rb = buf(numel), buf(numel)
    stream = torch.cuda.Stream()

    def body():
        comm.all_reduce(x, y)
        comm.all_gather(g_in, g_out)
        with group():
            for a, b in zip(small_in, small_out):
                comm.all_reduce(a, b, op="max")
        with group():
            comm.send(sb, (rank + 1) % n)
            comm.recv(rb, (rank - 1) % n)

    # a first eager pass (lazy set-up happens outside the capture), then the capture
    with torch.cuda.stream(stream):
        body()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        body()
    bad = []
    for it in range(10):
        def val(p, k):
            return float(1 + p + 10 * it + k)
        x.fill_(val(rank, 0))
        g_in.fill_(val(rank, 1))
        for i, a in enumerate(small_in):
            a.fill_(val(rank, 2 + i))
        sb.fill_(val(rank, 20))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        if not torch.all(y == sum(val(p, 0) for p in range(n))):
            bad.append((it, "all_reduce"))
        for p in range(n):
            if not torch.all(g_out[p * numel:(p + 1) * numel] == val(p, 1)):
                bad.append((it, "all_gather", p))
        for i, b in enumerate(small_out):
            if not torch.all(b == max(val(p, 2 + i) for p in range(n))):
                bad.append((it, "grouped all_reduce", i))
        if not torch.all(rb == val((rank - 1) % n, 20)):
            bad.append((it, "sendrecv"))
    err = comm.async_error()
    comm.destroy()
    return {"bad": bad, "err": err}


def test_capture_and_replay_one_rank():
    if _ngpus() < 1:
        pytest.skip("needs a GPU")
    res = run_ranks(_capture_rank, 1, args=(False,), timeout=300)
    assert res[0]["bad"] == [] and res[0]["err"] == 0, res[0]


@pytest.mark.parametrize("registered", [True, False])
def test_capture_and_replay_two_ranks(registered):
    if _ngpus() < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_capture_rank, 2, args=(registered,), timeout=300)
    for r in range(2):
        assert res[r]["bad"] == [] and res[r]["err"] == 0, res[r]
