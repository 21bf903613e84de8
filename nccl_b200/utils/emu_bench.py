"""Times the collective kernels in single-GPU emulation: one cooperative grid plays all ranks
(rank = blockIdx.y), so the protocols (flags, barriers, reductions) run exactly as between GPUs
but every "remote" access stays on this device. Useful to profile a kernel's own overheads.

    python -m nccl_b200.utils.emu_bench --ranks 4 --count 262144 --kernel p2p --ctas 16 --iters 100
"""
import argparse
import ctypes
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--count", type=int, default=262144, help="fp32 elements per rank")
    ap.add_argument("--kernel", default="p2p", choices=("p2p", "ll"))
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
    kernel = 0 if a.kernel == "p2p" else 1

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
    ref = sum(ins)
    err = (outs[0] - ref).abs().max().item()
    print("emulated all-reduce: ranks %d count %d kernel %s ctas %d: %.2f us per launch, max error %.2e" %
          (n, a.count, a.kernel, a.ctas, e0.elapsed_time(e1) * 1e3 / a.iters, err), flush=True)
    lib.b200EmuDestroy(ctx)
    return 0


if __name__ == "__main__":
    sys.exit(main())
