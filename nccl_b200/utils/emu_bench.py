"""Times the collective kernels in single-GPU emulation: one cooperative grid plays all ranks
(rank = blockIdx.y), so the protocols (flags, barriers, reductions) run exactly as between GPUs
but every "remote" access stays on this device. Useful to profile a kernel's own overheads.

    python -m nccl_b200.utils.emu_bench --ranks 4 --count 262144 --kernel p2p --ctas 16 --iters 100
    python -m nccl_b200.utils.emu_bench --ranks 4 --count 262144 --kernel push        # all-gather: push | pull | bpush | bpull | llcopy
    python -m nccl_b200.utils.emu_bench --ranks 4 --count 262144 --kernel sendrecv    # ring of grouped send / receive
"""
import argparse
import ctypes
import sys

import torch

MODE_PUSH, MODE_PULL, MODE_LL = 0, 1, 3   # copy-kernel variants of the emulation entry point


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--count", type=int, default=262144, help="fp32 elements per rank")
    ap.add_argument("--kernel", default="p2p", choices=("p2p", "ll", "push", "pull", "bpush", "bpull", "llcopy", "sendrecv"),
                    help="p2p / ll: all-reduce kernels; push / pull / llcopy: all-gather through the copy kernels (bpush / bpull: moved by the bulk-copy engines); sendrecv: mailbox ring")
    ap.add_argument("--ctas", type=int, default=16)
    ap.add_argument("--iters", type=int, default=100)
    a = ap.parse_args(argv)
    from nccl_b200 import _lib, core
    lib = _lib.load()
    lib.b200EmuCreate.restype = ctypes.c_void_p
    lib.b200EmuCreate.argtypes = [ctypes.c_int, ctypes.c_ulonglong]
    lib.b200EmuDestroy.argtypes = [ctypes.c_void_p]
    lib.b200EmuReduce.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t,
                                  ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int]
    n = a.ranks
    ctx = lib.b200EmuCreate(n, 5000)
    ins = [torch.randn(a.count, device="cuda") for _ in range(n)]
    outs = [torch.zeros(a.count, device="cuda") for _ in range(n)]
    pin = (ctypes.c_void_p * n)(*[t.data_ptr() for t in ins])
    pout = (ctypes.c_void_p * n)(*[t.data_ptr() for t in outs])
    lib.b200EmuCopy.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p),
                                ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int]
    lib.b200EmuP2p.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                               ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_size_t), ctypes.c_int]
    kernel = 0 if a.kernel == "p2p" else 1
    nbytes = a.count * 4
    if a.kernel in ("push", "pull", "bpush", "bpull", "llcopy"):
        gathered = [torch.zeros(a.count * n, device="cuda") for _ in range(n)]
        pgat = (ctypes.c_void_p * n)(*[t.data_ptr() for t in gathered])
        mode = {"push": MODE_PUSH, "pull": MODE_PULL, "bpush": MODE_PUSH | 4, "bpull": MODE_PULL | 4, "llcopy": MODE_LL}[a.kernel]

        def call():
            rc = lib.b200EmuCopy(ctx, 2, mode, nbytes, pin, pgat, 0, a.ctas)   # 2 = all-gather
            assert rc == 0, rc
    elif a.kernel == "sendrecv":
        ranks, peers, sends, bufs, sizes = [], [], [], [], []
        for r in range(n):
            ranks += [r, r]
            peers += [(r + 1) % n, (r - 1) % n]
            sends += [1, 0]
            bufs += [ins[r].data_ptr(), outs[r].data_ptr()]
            sizes += [nbytes, nbytes]
        k = len(ranks)
        c_int = ctypes.c_int * k
        args = (k, c_int(*ranks), c_int(*peers), c_int(*sends), (ctypes.c_void_p * k)(*bufs), (ctypes.c_size_t * k)(*sizes), max(1, min(a.ctas, 4)))

        def call():
            rc = lib.b200EmuP2p(ctx, *args)
            assert rc == 0, rc
    else:
        def call():
            rc = lib.b200EmuReduce(ctx, kernel, 4, core.FP32, 0, a.count, pin, pout, 0, a.ctas)   # 4 = all-reduce, op 0 = sum
            assert rc == 0, rc

    for _ in range(3):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        call()
    e1.record()
    torch.cuda.synchronize()
    if a.kernel in ("push", "pull", "bpush", "bpull", "llcopy"):
        err = (gathered[n - 1] - torch.cat(ins)).abs().max().item()
    elif a.kernel == "sendrecv":
        err = (outs[0] - ins[n - 1]).abs().max().item()
    else:
        err = (outs[0] - sum(ins)).abs().max().item()
    print("emulated %s: ranks %d count %d kernel %s ctas %d: %.2f us per launch, max error %.2e" %
          ("all-reduce" if a.kernel in ("p2p", "ll") else "all-gather" if a.kernel != "sendrecv" else "send/recv ring", n, a.count, a.kernel, a.ctas,
           e0.elapsed_time(e1) * 1e3 / a.iters, err), flush=True)
    lib.b200EmuDestroy(ctx)
    return 0


if __name__ == "__main__":
    sys.exit(main())
