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


@pytest.mark.parametrize("n,E,K,H,T", [(2, 4, 2, 128, 5), (4, 8, 2, 256, 16), (8, 32, 4, 512, 33), (8, 256, 8, 1024, 64), (2, 4, 2, 128, 300)])
@pytest.mark.parametrize("fp8", [0, 1])
@pytest.mark.parametrize("bulk", [1, 0])
def test_dispatch_combine(n, E, K, H, T, fp8, bulk):
    """bulk=1: the packed tokens leave through the bulk-copy engines from a ring of shared-memory stages (33 and 64
    tokens over 4 CTAs wrap the ring several times); bulk=0: the warps store them. 300 tokens over 4 CTAs: more tokens per
    CTA than the combine stages routing data for in shared memory, so both of its paths run."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    lib = _lib()
    lib.b200EpEmuBulk.argtypes = [ctypes.c_void_p, ctypes.c_int]
    El, cap = E // n, n * T
    ctx = lib.b200EpEmuCreate(n, E, K, H, T)
    assert ctx
    assert lib.b200EpEmuBulk(ctx, bulk) == 0
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


def _lib2():
    lib = _lib()
    lib.b200EpEmuSet.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_int, ctypes.c_ulonglong]
    lib.b200EpEmuMask.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_uint)]
    lib.b200EpEmuClear.argtypes = [ctypes.c_void_p]
    return lib


def _batch(n, E, K, H, T, g):
    x = [torch.randn(T, H, generator=g).bfloat16().cuda() for _ in range(n)]
    idx = [torch.rand(T, E, generator=g).topk(K, dim=1).indices.to(torch.int64).cuda() for _ in range(n)]
    wts = [torch.rand(T, K, generator=g).cuda() for _ in range(n)]
    return x, idx, wts


def test_split_phase_dispatch_and_combine():
    """send_only + complete: the sending half and the receiving half of each kernel run as two launches
    (whatever the caller queues in between overlaps the sends) and give the result of the one-launch call."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    lib = _lib2()
    n, E, K, H, T = 4, 16, 2, 256, 24
    El, cap = E // n, n * T
    ctx = lib.b200EpEmuCreate(n, E, K, H, T)
    assert ctx
    g = torch.Generator().manual_seed(5)
    try:
        for rep in range(3):
            x, idx, wts = _batch(n, E, K, H, T, g)
            ntok = (ctypes.c_int * n)(*([T] * n))
            out_tok = [torch.zeros(El, cap, H, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
            counts = [(ctypes.c_int * El)() for _ in range(n)]
            cptr = (ctypes.POINTER(ctypes.c_int) * n)(*[ctypes.cast(c, ctypes.POINTER(ctypes.c_int)) for c in counts])
            assert lib.b200EpEmuSet(ctx, 1, 0, 0, 0) == 0
            assert lib.b200EpEmuDispatch(ctx, 0, ntok, _ptrs(x), _ptrs(idx), _ptrs(out_tok), None, cptr, 4) == 0
            assert lib.b200EpEmuSet(ctx, 2, 0, 0, 0) == 0
            assert lib.b200EpEmuDispatch(ctx, 0, ntok, _ptrs(x), _ptrs(idx), _ptrs(out_tok), None, cptr, 3) == 0
            for r in range(n):
                for el in range(El):
                    e = r * El + el
                    assert counts[r][el] == sum(int((idx[s] == e).sum()) for s in range(n))
            outs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
            assert lib.b200EpEmuSet(ctx, 1, 0, 0, 0) == 0
            assert lib.b200EpEmuCombine(ctx, ntok, _ptrs(out_tok), _ptrs(idx), _ptrs(wts), _ptrs(outs), 4) == 0
            assert lib.b200EpEmuSet(ctx, 2, 0, 0, 0) == 0
            assert lib.b200EpEmuCombine(ctx, ntok, _ptrs(out_tok), _ptrs(idx), _ptrs(wts), _ptrs(outs), 2) == 0
            for r in range(n):
                ref = x[r].float() * wts[r].sum(1, keepdim=True)
                assert torch.allclose(outs[r].float(), ref, rtol=2e-2, atol=2e-2), (rep, r)
    finally:
        lib.b200EpEmuDestroy(ctx)


def test_rank_that_never_joins_is_masked_out():
    """One rank never shows up. Without masks its peers' waits run out and the call reports a time-out; with
    masks enabled the waits leave that rank out, the call completes with what the live ranks sent, the mask
    shows the missing rank, and later calls neither send to it nor wait for it (so they are fast again)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import time
    lib = _lib2()
    n, E, K, H, T = 4, 8, 2, 128, 8
    El, cap = E // n, n * T
    dead = 2
    ctx = lib.b200EpEmuCreate(n, E, K, H, T)
    assert ctx
    g = torch.Generator().manual_seed(9)
    try:
        x, idx, wts = _batch(n, E, K, H, T, g)
        ntok = (ctypes.c_int * n)(*([T] * n))
        out_tok = [torch.zeros(El, cap, H, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
        counts = [(ctypes.c_int * El)() for _ in range(n)]
        cptr = (ctypes.POINTER(ctypes.c_int) * n)(*[ctypes.cast(c, ctypes.POINTER(ctypes.c_int)) for c in counts])
        # masks off: the wait on the absent rank runs out (200 ms) and is reported
        assert lib.b200EpEmuSet(ctx, 3, 1 << dead, 0, 200) == 0
        assert lib.b200EpEmuDispatch(ctx, 0, ntok, _ptrs(x), _ptrs(idx), _ptrs(out_tok), None, cptr, 2) == 8   # ncclTimeout
        lib.b200EpEmuClear(ctx)
        lib.b200EpEmuDestroy(ctx)
        ctx = lib.b200EpEmuCreate(n, E, K, H, T)
        # masks on: same absence, the call completes
        assert lib.b200EpEmuSet(ctx, 3, 1 << dead, 1, 200) == 0
        assert lib.b200EpEmuDispatch(ctx, 0, ntok, _ptrs(x), _ptrs(idx), _ptrs(out_tok), None, cptr, 2) == 0
        live = [r for r in range(n) if r != dead]
        for r in live:
            m = (ctypes.c_uint * n)()
            assert lib.b200EpEmuMask(ctx, r, m) == 0
            assert [int(v != 0) for v in m] == [int(q == dead) for q in range(n)], (r, list(m))
            for el in range(El):
                e = r * El + el
                assert counts[r][el] == sum(int((idx[s] == e).sum()) for s in live)
        # combine: rows owned by the missing rank's experts are left out of the sums
        outs = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
        t0 = time.time()
        assert lib.b200EpEmuCombine(ctx, ntok, _ptrs(out_tok), _ptrs(idx), _ptrs(wts), _ptrs(outs), 2) == 0
        assert time.time() - t0 < 0.15, "a masked rank must not be waited for"
        for r in live:
            alive = ((idx[r] // El) != dead).float()
            ref = x[r].float() * (wts[r] * alive).sum(1, keepdim=True)
            assert torch.allclose(outs[r].float(), ref, rtol=2e-2, atol=2e-2), r
        # the next dispatch does not wait for the masked rank either
        t0 = time.time()
        assert lib.b200EpEmuDispatch(ctx, 0, ntok, _ptrs(x), _ptrs(idx), _ptrs(out_tok), None, cptr, 2) == 0
        assert time.time() - t0 < 0.15
    finally:
        lib.b200EpEmuDestroy(ctx)


@pytest.mark.parametrize("layout", [1, 2])
@pytest.mark.parametrize("n,E,K,H,T", [(2, 4, 2, 128, 7), (4, 16, 4, 256, 16), (8, 64, 8, 512, 24)])
@pytest.mark.parametrize("fp8", [0, 1])
@pytest.mark.parametrize("bulk", [1, 0])
def test_rank_major_and_flat_layouts(layout, n, E, K, H, T, fp8, bulk):
    """One copy of a token per destination rank (not per expert): rank-major puts it at row (source, token), flat packs
    the received tokens; the routing row travels with the token. The caller pre-reduces its local experts with the
    weights and combine sums one row per rank."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    lib = _lib2()
    lib.b200EpEmuLayout.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.POINTER(ctypes.c_void_p)] * 3
    lib.b200EpEmuBulk.argtypes = [ctypes.c_void_p, ctypes.c_int]
    El, cap = E // n, n * T
    ctx = lib.b200EpEmuCreate(n, E, K, H, T)
    assert ctx
    assert lib.b200EpEmuBulk(ctx, bulk) == 0
    g = torch.Generator().manual_seed(77 + layout + n)
    try:
        for rep in range(3):
            ntok = [T - (r % 2) for r in range(n)]
            x = [torch.randn(ntok[r], H, generator=g).bfloat16().cuda() for r in range(n)]
            idx = [torch.rand(ntok[r], E, generator=g).topk(K, dim=1).indices.to(torch.int64) for r in range(n)]
            for r in range(n):
                idx[r][0, 0] = -1          # an unused entry
            idx = [i.cuda() for i in idx]
            wts = [torch.rand(ntok[r], K, generator=g).cuda() for r in range(n)]
            out_tok = [torch.zeros(cap, H, dtype=torch.uint8 if fp8 else torch.bfloat16, device="cuda") for _ in range(n)]
            out_sc = [torch.zeros(cap, H // 128, device="cuda") for _ in range(n)]
            out_idx = [torch.full((cap, K), -7, dtype=torch.int64, device="cuda") for _ in range(n)]
            out_w = [torch.zeros(cap, K, device="cuda") for _ in range(n)]
            counts = [(ctypes.c_int * El)() for _ in range(n)]
            cptr = (ctypes.POINTER(ctypes.c_int) * n)(*[ctypes.cast(c, ctypes.POINTER(ctypes.c_int)) for c in counts])
            assert lib.b200EpEmuLayout(ctx, layout, _ptrs(out_idx), _ptrs(out_w), _ptrs(wts)) == 0
            assert lib.b200EpEmuDispatch(ctx, fp8, (ctypes.c_int * n)(*ntok), _ptrs(x), _ptrs(idx), _ptrs(out_tok), _ptrs(out_sc) if fp8 else None, cptr, 5) == 0
            y = []
            for r in range(n):
                if fp8:
                    tok = (out_tok[r].view(torch.float8_e4m3fn).float().view(cap, H // 128, 128) * out_sc[r].unsqueeze(-1)).view(cap, H)
                else:
                    tok = out_tok[r].float()
                valid = (out_idx[r] >= 0).any(1)
                # expected: which (source, token) pairs have an expert on rank r
                want = []
                for s in range(n):
                    loc = (idx[s] >= 0) & ((idx[s] // El) == r)
                    for t in torch.nonzero(loc.any(1)).flatten().tolist():
                        want.append((s, t))
                assert int(valid.sum()) == len(want), (r, int(valid.sum()), len(want))
                for el in range(El):
                    assert counts[r][el] == sum(int((idx[s] == r * El + el).sum()) for s in range(n))
                if layout == 1:
                    rows = [s * T + t for s, t in want]
                    assert sorted(torch.nonzero(valid).flatten().tolist()) == sorted(rows)
                    pairs = list(zip(rows, want))
                else:
                    # packed, grouped by source rank: rows [0, total) are in use; identify every row by its routing row + payload
                    total = len(want)
                    assert bool(valid[:total].all()) and not bool(valid[total:].any())
                    pairs, pos = [], 0
                    for s in range(n):
                        mine = [t for ss, t in want if ss == s]
                        block = tok[pos:pos + len(mine)]
                        ref = torch.stack([x[s][t].float() for t in mine]) if mine else block
                        if mine:
                            nearest = torch.cdist(block, ref).argmin(1).tolist()
                            assert sorted(nearest) == list(range(len(mine))), (r, s)
                            pairs += [(pos + i, (s, mine[j])) for i, j in enumerate(nearest)]
                        pos += len(mine)
                tol = 0.08 if fp8 else 0.0
                for row, (s, t) in pairs:
                    assert torch.allclose(tok[row], x[s][t].float(), rtol=tol, atol=2 * tol), (r, s, t)
                    loc = (idx[s][t] >= 0) & ((idx[s][t] // El) == r)
                    assert torch.equal(out_idx[r][row], torch.where(loc, idx[s][t], torch.full_like(idx[s][t], -1)))
                    assert torch.equal(out_w[r][row], wts[s][t])
                # the caller's part: expert e multiplies by (e + 1); local experts pre-reduced with the weights
                scale = (out_w[r] * (out_idx[r] + 1).clamp(min=0).float() * (out_idx[r] >= 0)).sum(1, keepdim=True)
                y.append((tok * scale).bfloat16().contiguous())
            outs = [torch.zeros(ntok[r], H, dtype=torch.bfloat16, device="cuda") for r in range(n)]
            assert lib.b200EpEmuCombine(ctx, (ctypes.c_int * n)(*ntok), _ptrs(y), _ptrs(idx), None, _ptrs(outs), 5) == 0
            for r in range(n):
                sc = (wts[r] * (idx[r] + 1).clamp(min=0).float() * (idx[r] >= 0)).sum(1, keepdim=True)
                ref = x[r].float() * sc
                tol = 0.1 if fp8 else 0.03
                assert torch.allclose(outs[r].float(), ref, rtol=tol, atol=tol * ref.abs().max().item()), (rep, r)
    finally:
        lib.b200EpEmuDestroy(ctx)
