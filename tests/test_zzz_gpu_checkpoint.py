"""Process-wide checkpoint calls on GPU communicators: ncclCheckpointPrepare releases the library's device memory
and peer mappings of every communicator of the process, ncclCheckpointRestore maps them again, and the same
communicator handles keep working."""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu


def _rank(rank, nranks, uid):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator, _lib
    comm = Communicator(nranks, rank, uid)
    lib = comm.lib
    x = torch.full((1 << 16,), float(rank + 1), device="cuda")
    comm.all_reduce(x)
    torch.cuda.synchronize()
    before = comm.mem_stats(0)
    _lib.check(lib.ncclCheckpointPrepare(), "ncclCheckpointPrepare", lib)
    suspended, left = comm.mem_stats(1), comm.mem_stats(0)
    _lib.check(lib.ncclCheckpointRestore(), "ncclCheckpointRestore", lib)
    y = torch.full((1 << 16,), float(rank + 1), device="cuda")
    comm.all_reduce(y)
    torch.cuda.synchronize()
    assert comm.async_error() == 0
    out = float(x[0]), float(y[0]), before, suspended, left, comm.mem_stats(1)
    comm.destroy()
    return out


def test_process_wide_prepare_restore_on_gpus():
    n = min(torch.cuda.device_count() if torch.cuda.is_available() else 0, 4)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_rank, n, timeout=200)
    tot = n * (n + 1) / 2
    for r in range(n):
        x, y, before, suspended, left, after = res[r]
        assert x == tot and y == tot
        assert before > 0 and suspended == 1 and left == 0 and after == 0
