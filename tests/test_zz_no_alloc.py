"""The allocation-free all-reduce entry point (b200NoAllocAllReduce).

Some callers cannot allocate device memory when they need a reduction (all memory already handed
to their own pool, or they run inside an allocator callback), so this entry point keeps its
working memory in a fixed array of the library image. The test calls it through its exported C
symbol, twice in a row (the second call finds the array as the first one left it), compares each
result with the regular flagged-line all-reduce of the library and with a plain fp32 sum computed by
PyTorch, and checks that every rank received identical bits, that the amount of free device memory
did not move and that oversized requests are refused. A second test changes the number of ranks
between calls (2, then 8, then 3), which the shared epoch word of the array has to survive.
This file sorts last so that a run stopping at the first failure has run everything else before.
"""
import ctypes

import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _ptrs(ts):
    return (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


@pytest.mark.parametrize("n,dtype,code,count", [(8, torch.float32, 7, 1024), (4, torch.bfloat16, 9, 2047), (2, torch.float16, 6, 5), (1, torch.float32, 7, 33)])
def test_no_alloc_allreduce_matches_regular_entry_point(n, dtype, code, count):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from nccl_b200 import _lib
    lib = _lib.load()
    fn = lib.b200NoAllocAllReduce
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
    lib.b200EmuCreate.restype = ctypes.c_void_p
    lib.b200EmuCreate.argtypes = [ctypes.c_int, ctypes.c_ulonglong]
    lib.b200EmuDestroy.argtypes = [ctypes.c_void_p]
    lib.b200EmuReduce.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t,
                                  ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int]
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(1234 + n)
    ctx = lib.b200EmuCreate(n, 5000)
    assert ctx
    try:
        # all buffers exist before the free-memory reading, and a first call has done the set-up
        ins = [[torch.randn(count, generator=g).to(dtype).cuda() for _ in range(n)] for _ in range(2)]
        got = [torch.zeros(count, dtype=dtype, device="cuda") for _ in range(n)]
        want = [torch.zeros(count, dtype=dtype, device="cuda") for _ in range(n)]
        assert fn(n, code, count, _ptrs(ins[0]), _ptrs(got), None) == 0
        torch.cuda.synchronize()
        for call in range(2):   # two calls in a row share the scratch array
            for t in got + want:
                t.zero_()
            torch.cuda.synchronize()
            # free memory is read directly around the call: what PyTorch's caching allocator does for the comparisons
            # below (it takes memory from the driver in 2 MiB segments) is not the entry point's doing
            free_before = torch.cuda.mem_get_info()[0]
            assert fn(n, code, count, _ptrs(ins[call]), _ptrs(got), None) == 0
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_before, "the entry point must not allocate device memory"
            assert lib.b200EmuReduce(ctx, 1, 4, code, 0, count, _ptrs(ins[call]), _ptrs(want), 0, 1) == 0
            torch.cuda.synchronize()
            tol = {torch.float32: 1e-6, torch.float16: 2 ** -10, torch.bfloat16: 2 ** -7}[dtype]
            ref = torch.stack([t.float() for t in ins[call]]).sum(0)   # plain fp32 sum of the same inputs
            for r in range(n):
                assert torch.allclose(got[r].float(), want[r].float(), rtol=tol, atol=tol), (call, r)
                assert torch.allclose(got[r].float(), ref, rtol=tol, atol=tol * n), (call, r)
                assert torch.equal(got[r], got[0]), "every rank must receive identical bits"
        # beyond the fixed scratch: refused, nothing launched
        es = torch.empty(0, dtype=dtype).element_size()
        assert fn(n, code, 4096 // es + 1, _ptrs(ins[0]), _ptrs(got), None) == 4   # ncclInvalidArgument
        assert fn(9, code, 1, _ptrs(ins[0]), _ptrs(got), None) == 4
    finally:
        lib.b200EmuDestroy(ctx)


def test_no_alloc_allreduce_survives_a_changing_rank_count():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from nccl_b200 import _lib
    lib = _lib.load()
    fn = lib.b200NoAllocAllReduce
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(99)
    count = 777
    for n in (2, 8, 3, 8, 1, 5):
        ins = [torch.randn(count, generator=g).cuda() for _ in range(n)]
        got = [torch.zeros(count, device="cuda") for _ in range(n)]
        assert fn(n, 7, count, _ptrs(ins), _ptrs(got), None) == 0, n
        torch.cuda.synchronize()
        ref = torch.stack(ins).sum(0)
        for r in range(n):
            assert torch.allclose(got[r], ref, rtol=1e-6, atol=1e-5), (n, r)
            assert torch.equal(got[r], got[0])
    # a count whose size in bytes wraps around must be refused, not reduced to one element
    assert fn(2, 7, (1 << 62) + 1, _ptrs(ins[:2]), _ptrs(got[:2]), None) == 4
