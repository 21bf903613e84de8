"""All-reduce of pinned host tensors through device staging, chunked and overlapped (ncclAllReduceFromHost)."""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402

pytestmark = pytest.mark.gpu


def _rank(rank, nranks, uid):
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    out = {}
    for case, (numel, dtype, chunk, in_place) in enumerate([((1 << 22) + 12345, torch.float32, 1 << 20, False), (3 << 20, torch.bfloat16, 0, True),
                                                            (1000, torch.float32, 4096, False)]):
        dev_in = torch.empty(numel, dtype=dtype, device="cuda")
        dev_out = dev_in if in_place else torch.empty(numel, dtype=dtype, device="cuda")
        hin = torch.empty(numel, dtype=dtype).pin_memory()
        hout = torch.empty(numel, dtype=dtype).pin_memory()
        errs = []
        for it in range(3):   # later calls reuse the chunk slots and their events
            g = torch.Generator().manual_seed(1000 * case + 10 * it + rank)
            hin.copy_(torch.randn(numel, generator=g).to(dtype))
            hout.zero_()
            comm.all_reduce_from_host(hin, hout, dev_in, dev_out, chunk_bytes=chunk)
            torch.cuda.current_stream().synchronize()   # the stream waits for the last copy out
            ref = sum(torch.randn(numel, generator=torch.Generator().manual_seed(1000 * case + 10 * it + r)).to(dtype).float() for r in range(nranks))
            errs.append(float((hout.float() - ref).abs().max()))
        out[case] = errs
    assert comm.async_error() == 0
    comm.destroy()
    return out


@pytest.mark.parametrize("n", [1, 2])
def test_all_reduce_from_host(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    res = run_ranks(_rank, n, timeout=180)
    for r in range(n):
        assert max(res[r][0]) < 1e-5 * n and max(res[r][2]) < 1e-5 * n, res[r]
        assert max(res[r][1]) < 0.05 * n, res[r]
