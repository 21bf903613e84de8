"""Expert-parallel dispatch / combine kernels on one GPU (all ranks played by one cooperative grid)."""
import ctypes

import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def _lib():
    from nccl_b200 import _lib
    lib = _lib.load()
    lib.b200EpEmuCreate.restype = ctypes.c_void_p
    lib.b200EpEmuCreate.argtypes = [ctypes.c_int] * 5
    lib.b200EpEmuDestroy.argtypes = [ctypes.c_void_p]
    pp = ctypes.POINTER(ctypes.c_void_p)
    lib.b200EpEmuDispatch.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int), pp, pp, pp, pp, ctypes.POINTER(ctypes.POINTER(ctypes.c_int)), ctypes.c_int]
    lib.b200EpEmuCombine.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), pp, pp, pp, pp, ctypes.c_int]
    return lib


def _ptrs(ts):
    return (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


@pytest.mark.parametrize("n,E,K,H,T", [(2, 4, 2, 128, 5), (4, 8, 2, 256, 16), (8, 32, 4, 512, 33), (8, 256, 8, 1024, 64)])
@pytest.mark.parametrize("fp8", [0, 1])
def test_dispatch_combine(n, E, K, H, T, fp8):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    lib = _lib()
    El, cap = E // n, n * T
    ctx = lib.b200EpEmuCreate(n, E, K, H, T)
    assert ctx
    g = torch.Generator().manual_seed(n * 1000 + E + K + fp8)
    try:
        for rep in range(3):   # landing zones alternate by call parity
            ntok = [T - (r % 3) for r in range(n)]
            x = [torch.randn(ntok[r], H, generator=g).bfloat16().cuda() for r in range(n)]
            idx = []
            for r in range(n):
                scores = torch.rand(ntok[r], E, generator=g)
                top = scores.topk(K, dim=1).indices.to(torch.int64)
                top[0, K - 1] = -1     # an unused entry
                idx.append(top.cuda())
            wts = [torch.rand(ntok[r], K, generator=g).cuda() for r in range(n)]
            out_dtype = torch.float8_e4m3fn if fp8 else torch.bfloat16
            out_tok = [torch.zeros(El, cap, H, dtype=torch.uint8 if fp8 else torch.bfloat16, device="cuda") for _ in range(n)]
            out_sc = [torch.zeros(El, cap, H // 128, device="cuda") for _ in range(n)]
            counts = [(ctypes.c_int * El)() for _ in range(n)]
            cptr = (ctypes.POINTER(ctypes.c_int) * n)(*[ctypes.cast(c, ctypes.POINTER(ctypes.c_int)) for c in counts])
            rc = lib.b200EpEmuDispatch(ctx, fp8, (ctypes.c_int * n)(*ntok), _ptrs(x), _ptrs(idx), _ptrs(out_tok), _ptrs(out_sc) if fp8 else None, cptr, 4)
            assert rc == 0
            # what every expert should have received, as a multiset of rows
            for r in range(n):
                for el in range(El):
                    e = r * El + el
                    want = [x[s][t].float() for s in range(n) for t in range(ntok[s]) for k in range(K) if int(idx[s][t, k]) == e]
                    cnt = counts[r][el]
                    assert cnt == len(want), (r, el, cnt, len(want))
                    if cnt == 0:
                        continue
                    if fp8:
                        got = out_tok[r][el, :cnt].view(out_dtype).float().view(cnt, H // 128, 128) * out_sc[r][el, :cnt].unsqueeze(-1)
                        got = got.view(cnt, H)
                    else:
                        got = out_tok[r][el, :cnt].float()
                    want = torch.stack(want).cuda()
                    # match rows irrespective of arrival order: nearest wanted row for every received row
                    nearest = torch.cdist(got, want).argmin(1)
                    assert sorted(nearest.tolist()) == list(range(cnt)), (r, el)
                    tol = 0.08 if fp8 else 0.0
                    assert torch.allclose(got, want[nearest], rtol=tol, atol=tol * 2), (r, el)
            if not fp8:
                # identity experts: combine must return x * (sum of the weights of the used entries)
                outs = [torch.zeros(ntok[r], H, dtype=torch.bfloat16, device="cuda") for r in range(n)]
                rc = lib.b200EpEmuCombine(ctx, (ctypes.c_int * n)(*ntok), _ptrs(out_tok), _ptrs(idx), _ptrs(wts), _ptrs(outs), 4)
                assert rc == 0
                for r in range(n):
                    wsum = (wts[r] * (idx[r] >= 0)).sum(1, keepdim=True)
                    ref = x[r].float() * wsum
                    assert torch.allclose(outs[r].float(), ref, rtol=2e-2, atol=2e-2), r
    finally:
        lib.b200EpEmuDestroy(ctx)
