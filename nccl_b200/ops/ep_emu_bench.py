"""Expert-parallel dispatch / combine kernels at a real shape on ONE GPU: one cooperative grid plays all ranks
(the emulation entry points of the library), so the kernels can be timed and profiled without a multi-GPU box.

    python -m nccl_b200.ops.ep_emu_bench --ranks 4 --tokens 1024 --hidden 7168 --experts 64 --topk 8 --layout expert_major

Prints one line with the device time of each kernel (CUDA events around the launch; the launch synchronises).
"""
import argparse
import ctypes

import torch

from .. import _lib


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--layout", default="expert_major", choices=("expert_major", "rank_major", "flat"))
    ap.add_argument("--fp8", type=int, default=1)
    ap.add_argument("--ctas", type=int, default=32, help="CTAs per emulated rank (ranks x ctas must fit the GPU)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--bulk", type=int, default=-1, help="1 / 0: dispatch through the bulk-copy engines or with the warps; -1: the library's default")
    a = ap.parse_args(argv)
    lib = _lib.load()
    pp = ctypes.POINTER(ctypes.c_void_p)
    lib.b200EpEmuCreate.restype = ctypes.c_void_p
    lib.b200EpEmuCreate.argtypes = [ctypes.c_int] * 5
    lib.b200EpEmuDestroy.argtypes = [ctypes.c_void_p]
    lib.b200EpEmuDispatch.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int), pp, pp, pp, pp, ctypes.POINTER(ctypes.POINTER(ctypes.c_int)), ctypes.c_int]
    lib.b200EpEmuCombine.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), pp, pp, pp, pp, ctypes.c_int]
    lib.b200EpEmuLayout.argtypes = [ctypes.c_void_p, ctypes.c_int, pp, pp, pp]
    lib.b200EpEmuBulk.argtypes = [ctypes.c_void_p, ctypes.c_int]
    n, E, K, H, T = a.ranks, a.experts, a.topk, a.hidden, a.tokens
    El, cap = E // n, n * T
    layout = {"expert_major": 0, "rank_major": 1, "flat": 2}[a.layout]
    ctx = lib.b200EpEmuCreate(n, E, K, H, T)
    assert ctx, "emulation context could not be created"
    lib.b200EpEmuBulk(ctx, a.bulk)
    ptrs = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])  # noqa: E731
    g = torch.Generator(device="cuda").manual_seed(1)
    x = [torch.randn(T, H, device="cuda", generator=g).bfloat16() for _ in range(n)]
    idx = [torch.rand(T, E, device="cuda", generator=g).topk(K, dim=1).indices.long().contiguous() for _ in range(n)]
    w = [torch.rand(T, K, device="cuda", generator=g) for _ in range(n)]
    rows = (El, cap) if layout == 0 else (cap,)
    toks = [torch.zeros(*rows, H, dtype=torch.uint8 if a.fp8 else torch.bfloat16, device="cuda") for _ in range(n)]
    scales = [torch.zeros(*rows, H // 128, device="cuda") for _ in range(n)]
    oidx = [torch.zeros(cap, K, dtype=torch.int64, device="cuda") for _ in range(n)]
    ow = [torch.zeros(cap, K, device="cuda") for _ in range(n)]
    y = [torch.zeros(*rows, H, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    out = [torch.zeros(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    counts = [(ctypes.c_int * El)() for _ in range(n)]
    cptr = (ctypes.POINTER(ctypes.c_int) * n)(*[ctypes.cast(c, ctypes.POINTER(ctypes.c_int)) for c in counts])
    ntok = (ctypes.c_int * n)(*([T] * n))
    if layout:
        assert lib.b200EpEmuLayout(ctx, layout, ptrs(oidx), ptrs(ow), ptrs(w)) == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    disp, comb = [], []
    for _ in range(a.iters):
        e0.record()
        rc = lib.b200EpEmuDispatch(ctx, a.fp8, ntok, ptrs(x), ptrs(idx), ptrs(toks), ptrs(scales) if a.fp8 else None, cptr, a.ctas)
        e1.record()
        torch.cuda.synchronize()
        assert rc == 0, rc
        disp.append(e0.elapsed_time(e1) * 1e3)
        e0.record()
        rc = lib.b200EpEmuCombine(ctx, ntok, ptrs(y), ptrs(idx), None if layout else ptrs(w), ptrs(out), a.ctas)
        e1.record()
        torch.cuda.synchronize()
        assert rc == 0, rc
        comb.append(e0.elapsed_time(e1) * 1e3)
    lib.b200EpEmuDestroy(ctx)
    recv = sum(sum(c) for c in counts)
    print("emulated expert parallelism: ranks %d tokens %d hidden %d experts %d top-%d layout %s fp8 %d ctas %d bulk %d: dispatch %.1f us, combine %.1f us "
          "(best of %d; %d rows counted over all ranks)" % (n, T, H, E, K, a.layout, a.fp8, a.ctas, a.bulk, min(disp), min(comb), a.iters, recv))


if __name__ == "__main__":
    main()
