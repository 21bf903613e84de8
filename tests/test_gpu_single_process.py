"""One process driving several GPUs: ncclCommInitAll, then grouped collectives over all communicators
from a single thread (the usage of the reference's multi-device-per-thread examples)."""
import ctypes

import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def test_init_all_and_grouped_allreduce():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from nccl_b200 import _lib
    from nccl_b200.core import FP32
    lib = _lib.load()
    n = min(torch.cuda.device_count(), 4)
    comms = (_lib.ncclComm_t * n)()
    _lib.check(lib.ncclCommInitAll(comms, n, None), "ncclCommInitAll", lib)
    xs, streams = [], []
    for d in range(n):
        torch.cuda.set_device(d)
        xs.append(torch.full((1 << 16,), float(d + 1), device="cuda:%d" % d))
        streams.append(torch.cuda.Stream(device=d))
    for it in range(3):
        _lib.check(lib.ncclGroupStart(), "ncclGroupStart", lib)
        for d in range(n):
            torch.cuda.set_device(d)
            rc = lib.ncclAllReduce(xs[d].data_ptr(), xs[d].data_ptr(), xs[d].numel(), FP32, 0, comms[d], streams[d].cuda_stream)
            _lib.check(rc, "ncclAllReduce", lib)
        _lib.check(lib.ncclGroupEnd(), "ncclGroupEnd", lib)
    for d in range(n):
        torch.cuda.set_device(d)
        streams[d].synchronize()
    total = float(sum(range(1, n + 1)))
    for d in range(n):
        assert float(xs[d][0]) == total * n * n and float(xs[d][-1]) == total * n * n   # three rounds: s, s*n, s*n*n
    for d in range(n):
        torch.cuda.set_device(d)
        e = ctypes.c_int()
        assert lib.ncclCommGetAsyncError(comms[d], ctypes.byref(e)) == 0 and e.value == 0
        _lib.check(lib.ncclCommDestroy(comms[d]), "ncclCommDestroy", lib)
