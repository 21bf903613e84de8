"""Kernel numerics on one GPU: every rank of a communicator is played by one cooperative grid.

Each case compares the CUDA kernel against a plain PyTorch fp32 (fp64 for 64-bit types) reference
of the same operation, reduced in rank order and rounded once, which is the kernels' rounding model.
"""
import ctypes

import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

KERNEL_REDUCE_P2P, KERNEL_ALLREDUCE_LL = 0, 1
FUNC_BROADCAST, FUNC_REDUCE, FUNC_ALLGATHER, FUNC_REDUCESCATTER, FUNC_ALLREDUCE = 0, 1, 2, 3, 4
FUNC_ALLTOALL, FUNC_SCATTER, FUNC_GATHER = 8, 9, 10
MODE_PUSH, MODE_PULL = 0, 1
MODE_BULK = 4   # added to a mode: moved by the bulk-copy engines instead of by threads


@pytest.fixture(scope="module")
def emu_lib():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from nccl_b200 import _lib
    lib = _lib.load()
    lib.b200EmuCreate.restype = ctypes.c_void_p
    lib.b200EmuCreate.argtypes = [ctypes.c_int, ctypes.c_ulonglong]
    lib.b200EmuDestroy.argtypes = [ctypes.c_void_p]
    lib.b200EmuReduce.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t,
                                  ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int]
    lib.b200EmuCopy.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p),
                                ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int]
    lib.b200EmuP2p.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                               ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_size_t), ctypes.c_int]
    lib.b200EmuStatus.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_uint)]
    lib.b200EmuClearStatus.argtypes = [ctypes.c_void_p]
    return lib


def _ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() if t is not None else 0 for t in tensors])


def _types():
    from nccl_b200 import core
    t = {torch.float32: core.FP32, torch.bfloat16: core.BF16, torch.float16: core.FP16, torch.int32: core.INT32,
         torch.int64: core.INT64, torch.float64: core.FP64, torch.uint8: core.UINT8, torch.int8: core.INT8}
    if hasattr(torch, "float8_e4m3fn"):
        t[torch.float8_e4m3fn] = core.FP8_E4M3
        t[torch.float8_e5m2] = core.FP8_E5M2
    return t


def _make_inputs(n, count, dtype, seed, op):
    g = torch.Generator(device="cpu").manual_seed(seed)
    outs = []
    for r in range(n):
        if dtype.is_floating_point:
            if op == "prod":
                x = 1.0 + 0.25 * (torch.rand(count, generator=g) - 0.5)
            else:
                x = torch.randn(count, generator=g)
            if dtype in (getattr(torch, "float8_e4m3fn", None), getattr(torch, "float8_e5m2", None)):
                x = x.clamp(-2, 2)
            x = x.to(dtype)
        elif dtype == torch.uint8:
            x = torch.randint(0, 3 if op == "prod" else 25, (count,), generator=g, dtype=torch.int32).to(dtype)
        else:
            x = torch.randint(-3 if op == "prod" else -1000, 4 if op == "prod" else 1000, (count,), generator=g, dtype=torch.int64).to(dtype)
        outs.append(x.cuda())
    return outs


def _reference(inputs, op, dtype):
    """Rank-ordered reduction in the accumulation type of the kernels, rounded once."""
    n = len(inputs)
    if dtype.is_floating_point:
        acc_t = torch.float64 if dtype == torch.float64 else torch.float32
    else:
        acc_t = torch.int64
    acc = inputs[0].to(acc_t)
    for x in inputs[1:]:
        y = x.to(acc_t)
        if op in ("sum", "avg"):
            acc = acc + y
        elif op == "prod":
            acc = acc * y
        elif op == "max":
            acc = torch.maximum(acc, y)
        else:
            acc = torch.minimum(acc, y)
    if op == "avg":
        if dtype.is_floating_point:
            acc = acc * torch.tensor(1.0 / n, dtype=torch.float32).to(acc_t) if acc_t == torch.float32 else acc * (1.0 / n)
        else:
            acc = torch.div(acc, n, rounding_mode="trunc")
    if not dtype.is_floating_point and dtype != torch.int64:
        # integer results wrap like the device type
        bits = torch.iinfo(dtype).bits
        acc = acc & ((1 << bits) - 1)
        if dtype != torch.uint8:
            acc = torch.where(acc >= (1 << (bits - 1)), acc - (1 << bits), acc)
    return acc.to(dtype)


def _is_fp8(dtype):
    return dtype in (getattr(torch, "float8_e4m3fn", None), getattr(torch, "float8_e5m2", None))


def _close(got, want, dtype):
    if _is_fp8(dtype):
        # fp32 accumulation in rank order, one rounding to fp8: the reference rounds the same sum with
        # PyTorch's conversion, so results agree except where the two roundings break a tie differently
        # (one fp8 step: 2^-3 relative for e4m3, 2^-2 for e5m2)
        g, w = got.float(), want.float()
        step = 2 ** -3 if dtype == torch.float8_e4m3fn else 2 ** -2
        return bool(((g - w).abs() <= step * w.abs() + 2 ** -9).all())
    if not dtype.is_floating_point or dtype in (torch.float32, torch.float64):
        # identical accumulation order and type: only fused multiply-add contraction can differ
        if dtype.is_floating_point:
            return torch.allclose(got.double(), want.double(), rtol=1e-6, atol=1e-6)
        return torch.equal(got, want)
    g, w = got.float(), want.float()
    # 16/8-bit floats: the fp32 accumulation is identical, so at most one rounding step apart
    tol = {torch.bfloat16: 2 ** -7, torch.float16: 2 ** -10}.get(dtype, 2 ** -2)
    return torch.allclose(g, w, rtol=tol, atol=tol)


OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}

REDUCE_CASES = [
    # (ranks, dtype, op, count)
    (2, torch.float32, "sum", 1 << 20),
    (8, torch.float32, "sum", (1 << 18) + 3),
    (8, torch.bfloat16, "sum", (1 << 20) + 5),
    (4, torch.float16, "sum", 4097),
    (3, torch.float32, "max", 1000),
    (5, torch.bfloat16, "min", 777),
    (8, torch.float32, "prod", 4096),
    (8, torch.float32, "avg", 12345),
    (4, torch.int32, "sum", 9999),
    (4, torch.int32, "avg", 1024),
    (7, torch.int64, "max", 513),
    (2, torch.float64, "sum", 2049),
    (8, torch.uint8, "sum", 100001),
    (8, torch.int8, "min", 333),
    (2, torch.float32, "sum", 1),
    (8, torch.bfloat16, "sum", 7),
    (8, torch.float16, "max", 30001),
    (3, torch.float64, "min", 4099),
    (5, torch.int64, "sum", 20011),
    (8, torch.float64, "avg", 1025),
    (6, torch.int64, "prod", 301),
] + ([
    (8, torch.float8_e4m3fn, "sum", 65543),
    (4, torch.float8_e5m2, "sum", 4099),
    (3, torch.float8_e4m3fn, "max", 1000),
    (8, torch.float8_e5m2, "min", 515),
] if hasattr(torch, "float8_e4m3fn") else [])


@pytest.mark.parametrize("n,dtype,op,count", REDUCE_CASES)
@pytest.mark.parametrize("kernel", [KERNEL_REDUCE_P2P, KERNEL_ALLREDUCE_LL])
def test_allreduce(emu_lib, n, dtype, op, count, kernel):
    es = torch.empty(0, dtype=dtype).element_size()
    if kernel == KERNEL_ALLREDUCE_LL and count * es > 256 * 1024:
        count = 256 * 1024 // es - 3
    ctx = emu_lib.b200EmuCreate(n, 5000)
    assert ctx
    try:
        ins = _make_inputs(n, count, dtype, 11 + n, op)
        want = _reference(ins, op, dtype)
        for rep in range(3):  # epochs and flag buffers are reused across calls
            outs = [torch.empty(count, dtype=dtype, device="cuda") for _ in range(n)]
            for o in outs:
                o.view(torch.uint8).zero_()
            ctas = 4 if kernel == KERNEL_REDUCE_P2P else min(16, max(1, (count * es + 4095) // 4096))
            rc = emu_lib.b200EmuReduce(ctx, kernel, FUNC_ALLREDUCE, _types()[dtype], OPS[op], count, _ptrs(ins), _ptrs(outs), 0, ctas)
            assert rc == 0
            for r in range(n):
                assert _close(outs[r], want, dtype), "rank %d rep %d" % (r, rep)
            assert all(torch.equal(outs[0].view(torch.uint8), o.view(torch.uint8)) for o in outs), "ranks disagree bit-wise"
    finally:
        emu_lib.b200EmuDestroy(ctx)


@pytest.mark.parametrize("n,dtype,op,count", [(8, torch.bfloat16, "sum", 4096), (4, torch.float32, "sum", 1001), (3, torch.float16, "max", 64)])
def test_allreduce_in_place_and_misaligned(emu_lib, n, dtype, op, count):
    ctx = emu_lib.b200EmuCreate(n, 5000)
    try:
        base = [torch.zeros(count + 8, dtype=dtype, device="cuda") for _ in range(n)]
        ins = _make_inputs(n, count, dtype, 3, op)
        for off in (0, 1):  # offset 1 element: not 16-byte aligned, exercises the element-wise path
            bufs = [b[off:off + count] for b in base]
            for b, x in zip(bufs, ins):
                b.copy_(x)
            want = _reference(ins, op, dtype)
            rc = emu_lib.b200EmuReduce(ctx, KERNEL_REDUCE_P2P, FUNC_ALLREDUCE, _types()[dtype], OPS[op], count, _ptrs(bufs), _ptrs(bufs), 0, 3)
            assert rc == 0
            for b in bufs:
                assert _close(b, want, dtype)
    finally:
        emu_lib.b200EmuDestroy(ctx)


@pytest.mark.parametrize("n,dtype,count", [(8, torch.bfloat16, 8192), (4, torch.float32, 1000), (2, torch.float32, 3), (5, torch.int32, 257)])
def test_reduce_scatter_and_reduce(emu_lib, n, dtype, count):
    ctx = emu_lib.b200EmuCreate(n, 5000)
    try:
        ins = _make_inputs(n, count * n, dtype, 5, "sum")
        want = _reference(ins, "sum", dtype)
        outs = [torch.zeros(count, dtype=dtype, device="cuda") for _ in range(n)]
        rc = emu_lib.b200EmuReduce(ctx, KERNEL_REDUCE_P2P, FUNC_REDUCESCATTER, _types()[dtype], 0, count, _ptrs(ins), _ptrs(outs), 0, 2)
        assert rc == 0
        for r in range(n):
            assert _close(outs[r], want[r * count:(r + 1) * count], dtype)
        root = n - 1
        full = [torch.zeros(count * n, dtype=dtype, device="cuda") for _ in range(n)]
        rc = emu_lib.b200EmuReduce(ctx, KERNEL_REDUCE_P2P, FUNC_REDUCE, _types()[dtype], 0, count * n, _ptrs(ins), _ptrs(full), root, 2)
        assert rc == 0
        assert _close(full[root], want, dtype)
        assert all(int(full[r].view(torch.uint8).max()) == 0 for r in range(n) if r != root)
    finally:
        emu_lib.b200EmuDestroy(ctx)


@pytest.mark.parametrize("n", [3, 4, 8])
@pytest.mark.parametrize("nbytes", [16, 48, 4096 + 16, (1 << 20) + 48, 3 << 20])
@pytest.mark.parametrize("ctas", [1, 5])
def test_broadcast_shared_out(emu_lib, n, nbytes, ctas):
    """Large-broadcast form: every non-root rank pulls one share of the root's buffer and stores it to all non-root
    ranks; the root copies its own output. In place and out of place, several launches (barrier epochs carry over)."""
    MODE_SPLIT_EMU = 8
    ctx = emu_lib.b200EmuCreate(n, 5000)
    try:
        g = torch.Generator().manual_seed(nbytes + n)
        for it, root in enumerate([n - 1, 0, 1]):
            send = [torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8).cuda() for _ in range(n)]
            recv = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(n)]
            if it == 2:
                recv[root] = send[root]   # in place on the root
            want = send[root].clone()
            assert emu_lib.b200EmuCopy(ctx, FUNC_BROADCAST, MODE_SPLIT_EMU, nbytes, _ptrs(send), _ptrs(recv), root, ctas) == 0
            torch.cuda.synchronize()
            assert all(torch.equal(r, want) for r in recv), (it, root)
    finally:
        emu_lib.b200EmuDestroy(ctx)


@pytest.mark.parametrize("n", [2, 3, 8])
@pytest.mark.parametrize("mode", [MODE_PUSH, MODE_PULL, MODE_PUSH | MODE_BULK, MODE_PULL | MODE_BULK])
@pytest.mark.parametrize("nbytes", [16, 4096 + 16, (1 << 20) + 48, 1001])
def test_copy_collectives(emu_lib, n, mode, nbytes):
    if (mode & MODE_BULK) and nbytes % 16:
        pytest.skip("the bulk-copy kernel moves multiples of 16 bytes (the host picks the thread kernel otherwise)")
    ctx = emu_lib.b200EmuCreate(n, 5000)
    try:
        g = torch.Generator().manual_seed(nbytes + n)
        # all-gather
        send = [torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8).cuda() for _ in range(n)]
        recv = [torch.zeros(nbytes * n, dtype=torch.uint8, device="cuda") for _ in range(n)]
        assert emu_lib.b200EmuCopy(ctx, FUNC_ALLGATHER, mode, nbytes, _ptrs(send), _ptrs(recv), 0, 3) == 0
        want = torch.cat(send)
        assert all(torch.equal(r, want) for r in recv)
        # all-to-all
        send = [torch.randint(0, 256, (nbytes * n,), generator=g, dtype=torch.uint8).cuda() for _ in range(n)]
        recv = [torch.zeros(nbytes * n, dtype=torch.uint8, device="cuda") for _ in range(n)]
        assert emu_lib.b200EmuCopy(ctx, FUNC_ALLTOALL, mode, nbytes, _ptrs(send), _ptrs(recv), 0, 3) == 0
        for r in range(n):
            want = torch.cat([send[p][r * nbytes:(r + 1) * nbytes] for p in range(n)])
            assert torch.equal(recv[r], want)
        # broadcast from the last rank
        root = n - 1
        send = [torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8).cuda() for _ in range(n)]
        recv = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(n)]
        assert emu_lib.b200EmuCopy(ctx, FUNC_BROADCAST, mode, nbytes, _ptrs(send), _ptrs(recv), root, 2) == 0
        assert all(torch.equal(r, send[root]) for r in recv)
        # scatter (push: root stores; pull: everyone loads its block from the root)
        send = [torch.randint(0, 256, (nbytes * n,), generator=g, dtype=torch.uint8).cuda() for _ in range(n)]
        recv = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(n)]
        assert emu_lib.b200EmuCopy(ctx, FUNC_SCATTER, mode, nbytes, _ptrs(send), _ptrs(recv), 0, 2) == 0
        for r in range(n):
            assert torch.equal(recv[r], send[0][r * nbytes:(r + 1) * nbytes])
        # gather to rank 0
        send = [torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8).cuda() for _ in range(n)]
        recv = [torch.zeros(nbytes * n, dtype=torch.uint8, device="cuda") for _ in range(n)]
        assert emu_lib.b200EmuCopy(ctx, FUNC_GATHER, mode, nbytes, _ptrs(send), _ptrs(recv), 0, 2) == 0
        assert torch.equal(recv[0], torch.cat(send))
    finally:
        emu_lib.b200EmuDestroy(ctx)


@pytest.mark.parametrize("n,nbytes", [(2, 1000), (4, (5 << 20) + 13), (8, 1 << 20)])
def test_send_recv_ring(emu_lib, n, nbytes):
    """Every rank sends to its successor and receives from its predecessor, twice (slot reuse)."""
    ctx = emu_lib.b200EmuCreate(n, 5000)
    try:
        g = torch.Generator().manual_seed(n)
        for rep in range(2):
            send = [torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8).cuda() for _ in range(n)]
            recv = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(n)]
            ranks, peers, sends, bufs, sizes = [], [], [], [], []
            for r in range(n):
                ranks += [r, r]
                peers += [(r + 1) % n, (r - 1) % n]
                sends += [1, 0]
                bufs += [send[r], recv[r]]
                sizes += [nbytes, nbytes]
            k = len(ranks)
            rc = emu_lib.b200EmuP2p(ctx, k, (ctypes.c_int * k)(*ranks), (ctypes.c_int * k)(*peers), (ctypes.c_int * k)(*sends),
                                    _ptrs(bufs), (ctypes.c_size_t * k)(*sizes), 2)
            assert rc == 0
            for r in range(n):
                assert torch.equal(recv[r], send[(r - 1) % n]), "rank %d rep %d" % (r, rep)
    finally:
        emu_lib.b200EmuDestroy(ctx)


def test_send_recv_several_per_peer(emu_lib):
    """Several sends to the same peer in one group arrive in posting order (sizes of less than one,
    exactly one and several mailbox chunks), and the next group continues the sequence."""
    n = 2
    ctx = emu_lib.b200EmuCreate(n, 5000)
    try:
        g = torch.Generator().manual_seed(7)
        sizes_each = [100, 1 << 20, (3 << 20) + 5, 16, 2 << 20]
        for rep in range(2):
            send = [[torch.randint(0, 256, (s,), generator=g, dtype=torch.uint8).cuda() for s in sizes_each] for _ in range(n)]
            recv = [[torch.zeros(s, dtype=torch.uint8, device="cuda") for s in sizes_each] for _ in range(n)]
            ranks, peers, sends, bufs, sizes = [], [], [], [], []
            for r in range(n):
                for i, s in enumerate(sizes_each):
                    ranks += [r, r]
                    peers += [1 - r, 1 - r]
                    sends += [1, 0]
                    bufs += [send[r][i], recv[r][i]]
                    sizes += [s, s]
            k = len(ranks)
            rc = emu_lib.b200EmuP2p(ctx, k, (ctypes.c_int * k)(*ranks), (ctypes.c_int * k)(*peers), (ctypes.c_int * k)(*sends),
                                    _ptrs(bufs), (ctypes.c_size_t * k)(*sizes), 1)
            assert rc == 0
            st = (ctypes.c_uint * 4)()
            assert emu_lib.b200EmuStatus(ctx, 0, st) == 0 and st[0] == 0
            for r in range(n):
                for i in range(len(sizes_each)):
                    assert torch.equal(recv[r][i], send[1 - r][i]), "rank %d op %d rep %d" % (r, i, rep)
    finally:
        emu_lib.b200EmuDestroy(ctx)


def test_wait_runs_out_and_reports(emu_lib):
    """A receive whose sender never posts: the wait gives up after its budget, the kernel returns
    and the status words say what it was waiting for. Nothing faults and the context stays usable."""
    ctx = emu_lib.b200EmuCreate(2, 200)  # 200 ms budget per wait
    try:
        buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
        rc = emu_lib.b200EmuP2p(ctx, 1, (ctypes.c_int * 1)(0), (ctypes.c_int * 1)(1), (ctypes.c_int * 1)(0), _ptrs([buf]),
                                (ctypes.c_size_t * 1)(4096), 1)
        assert rc == 0
        st = (ctypes.c_uint * 4)()
        assert emu_lib.b200EmuStatus(ctx, 0, st) == 0
        assert st[0] == 1          # DEV_TIMEOUT
        assert st[1] == 3          # waiting for a mailbox ready flag
        assert st[2] == 1          # of rank 1
        # the device is still usable
        assert int((torch.ones(8, device="cuda") * 2).sum().item()) == 16
    finally:
        emu_lib.b200EmuDestroy(ctx)


@pytest.mark.parametrize("n,dtype,count", [(8, torch.bfloat16, 1024), (4, torch.float32, 1001), (3, torch.float16, 5), (2, torch.int32, 4099)])
def test_flagged_line_reduce_scatter_and_reduce(emu_lib, n, dtype, count):
    ctx = emu_lib.b200EmuCreate(n, 5000)
    try:
        for rep in range(3):
            ins = _make_inputs(n, count * n, dtype, 21 + rep, "sum")
            want = _reference(ins, "sum", dtype)
            outs = [torch.zeros(count, dtype=dtype, device="cuda") for _ in range(n)]
            assert emu_lib.b200EmuReduce(ctx, KERNEL_ALLREDUCE_LL, FUNC_REDUCESCATTER, _types()[dtype], 0, count, _ptrs(ins), _ptrs(outs), 0, 2) == 0
            for r in range(n):
                assert _close(outs[r], want[r * count:(r + 1) * count], dtype), (rep, r)
            root = rep % n
            full = [torch.zeros(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            assert emu_lib.b200EmuReduce(ctx, KERNEL_ALLREDUCE_LL, FUNC_REDUCE, _types()[dtype], 0, count * n, _ptrs(ins), _ptrs(full), root, 2) == 0
            assert _close(full[root], want, dtype)
    finally:
        emu_lib.b200EmuDestroy(ctx)


@pytest.mark.parametrize("n", [2, 5, 8])
@pytest.mark.parametrize("nbytes", [8, 13, 4096, 100003])
def test_flagged_line_copy_collectives(emu_lib, n, nbytes):
    MODE_LL = 3
    ctx = emu_lib.b200EmuCreate(n, 5000)
    try:
        g = torch.Generator().manual_seed(nbytes * 3 + n)

        def rnd(k):
            return torch.randint(0, 256, (k,), generator=g, dtype=torch.uint8).cuda()
        for rep in range(2):
            send = [rnd(nbytes) for _ in range(n)]
            recv = [torch.zeros(nbytes * n, dtype=torch.uint8, device="cuda") for _ in range(n)]
            assert emu_lib.b200EmuCopy(ctx, FUNC_ALLGATHER, MODE_LL, nbytes, _ptrs(send), _ptrs(recv), 0, 2) == 0
            assert all(torch.equal(r, torch.cat(send)) for r in recv)
            send = [rnd(nbytes * n) for _ in range(n)]
            recv = [torch.zeros(nbytes * n, dtype=torch.uint8, device="cuda") for _ in range(n)]
            assert emu_lib.b200EmuCopy(ctx, FUNC_ALLTOALL, MODE_LL, nbytes, _ptrs(send), _ptrs(recv), 0, 2) == 0
            for r in range(n):
                assert torch.equal(recv[r], torch.cat([send[p][r * nbytes:(r + 1) * nbytes] for p in range(n)]))
            root = (rep + 1) % n
            send = [rnd(nbytes) for _ in range(n)]
            recv = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(n)]
            assert emu_lib.b200EmuCopy(ctx, FUNC_BROADCAST, MODE_LL, nbytes, _ptrs(send), _ptrs(recv), root, 1) == 0
            assert all(torch.equal(r, send[root]) for r in recv)
            send = [rnd(nbytes * n) for _ in range(n)]
            recv = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(n)]
            assert emu_lib.b200EmuCopy(ctx, FUNC_SCATTER, MODE_LL, nbytes, _ptrs(send), _ptrs(recv), root, 1) == 0
            for r in range(n):
                assert torch.equal(recv[r], send[root][r * nbytes:(r + 1) * nbytes])
            send = [rnd(nbytes) for _ in range(n)]
            recv = [torch.zeros(nbytes * n, dtype=torch.uint8, device="cuda") for _ in range(n)]
            assert emu_lib.b200EmuCopy(ctx, FUNC_GATHER, MODE_LL, nbytes, _ptrs(send), _ptrs(recv), root, 1) == 0
            assert torch.equal(recv[root], torch.cat(send))
    finally:
        emu_lib.b200EmuDestroy(ctx)


def _sweep_counts():
    return list(range(0, 261, 13)) + [1, 2, 3, 7, 8, 9, 15, 16, 17, 255, 256, 257] + list(range(4090, 4101))


@pytest.mark.parametrize("n", [2, 3, 5, 8])
@pytest.mark.parametrize("kernel", [KERNEL_REDUCE_P2P, KERNEL_ALLREDUCE_LL])
def test_allreduce_count_and_alignment_sweep(emu_lib, n, kernel):
    """Small counts (0 ... 260 and around 4096) at byte offsets 0 / 2 / 4 / 8 of the inputs and outputs,
    bf16 and fp32, with a band of a poison pattern on either side of every output: the kernel must
    write exactly the requested elements."""
    ctx = emu_lib.b200EmuCreate(n, 5000)
    assert ctx
    POISON = 0x5A
    try:
        for dtype in (torch.bfloat16, torch.float32):
            es = torch.empty(0, dtype=dtype).element_size()
            for count in sorted(set(_sweep_counts())):
                if count == 0:
                    continue   # the public API returns before launching anything for empty messages
                for off_bytes in (0, 2, 4, 8):
                    if off_bytes % es:
                        continue
                    off = off_bytes // es
                    band = 64 // es
                    src = _make_inputs(n, count, dtype, 1000 + count + off, "sum")
                    ins_base = [torch.zeros(count + off + band, dtype=dtype, device="cuda") for _ in range(n)]
                    ins = [b[off:off + count] for b in ins_base]
                    for b, x in zip(ins, src):
                        b.copy_(x)
                    outs_base = [torch.empty(band + off + count + band, dtype=dtype, device="cuda") for _ in range(n)]
                    for b in outs_base:
                        b.view(torch.uint8).fill_(POISON)
                    outs = [b[band + off:band + off + count] for b in outs_base]
                    ctas = 2 if kernel == KERNEL_REDUCE_P2P else 1
                    rc = emu_lib.b200EmuReduce(ctx, kernel, FUNC_ALLREDUCE, _types()[dtype], 0, count, _ptrs(ins), _ptrs(outs), 0, ctas)
                    assert rc == 0, (count, off_bytes)
                    want = _reference(src, "sum", dtype)
                    for r in range(n):
                        assert _close(outs[r], want, dtype), (str(dtype), count, off_bytes, r)
                        raw = outs_base[r].view(torch.uint8)
                        lo = (band + off) * es
                        hi = lo + count * es
                        assert bool((raw[:lo] == POISON).all()) and bool((raw[hi:] == POISON).all()), ("wrote outside", str(dtype), count, off_bytes, r)
    finally:
        emu_lib.b200EmuDestroy(ctx)


@pytest.mark.parametrize("n,dtype,op", [(8, torch.bfloat16, "sum"), (3, torch.float32, "max"), (5, torch.float16, "avg")])
def test_batched_allreduce_one_launch(emu_lib, n, dtype, op):
    """A group of small all-reduces (ragged counts, odd offsets) carried by one launch of the flagged-line kernel."""
    emu_lib.b200EmuReduceBatch.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_size_t),
                                           ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_void_p),
                                           ctypes.POINTER(ctypes.c_void_p), ctypes.c_int]
    ctx = emu_lib.b200EmuCreate(n, 5000)
    assert ctx
    try:
        es = torch.empty(0, dtype=dtype).element_size()
        counts = [1, 7, 2048, 3, 513, 4096, 33, 1000, 5, 2047] * 3
        offs, pos = [], 0
        for c in counts:
            offs.append(pos)
            pos += c + 3          # three elements of padding: items start at odd addresses
        total = pos
        for rep in range(2):
            ins = _make_inputs(n, total, dtype, 77 + rep, op)
            outs = [torch.zeros(total, dtype=dtype, device="cuda") for _ in range(n)]
            want = _reference(ins, op, dtype)
            ca = (ctypes.c_size_t * len(counts))(*counts)
            oa = (ctypes.c_size_t * len(counts))(*[o * es for o in offs])
            rc = emu_lib.b200EmuReduceBatch(ctx, _types()[dtype], OPS[op], len(counts), ca, oa, oa, _ptrs(ins), _ptrs(outs), 4)
            assert rc == 0
            for r in range(n):
                for c, o in zip(counts, offs):
                    assert _close(outs[r][o:o + c], want[o:o + c], dtype), (r, c, o)
                    assert bool((outs[r][o + c:o + c + 3].float() == 0).all()), "padding between items was written"
    finally:
        emu_lib.b200EmuDestroy(ctx)


def test_send_recv_small_and_mixed_sizes_many_rounds(emu_lib):
    """Forty rounds of a ring exchange whose size changes every round (1 byte ... 1 MiB, at odd offsets): small
    messages travel as flagged lines, larger ones through the chunked mailbox, and the per-pair sequence numbers,
    slot reuse and acknowledgements must stay in step across the two protocols."""
    n = 3
    ctx = emu_lib.b200EmuCreate(n, 5000)
    try:
        g = torch.Generator().manual_seed(17)
        sizes_cycle = [1, 8, 9, 16384, 16385, 100, 65536 + 3, 7, 16383, (1 << 20) + 5, 16, 3000, 4096]
        for rep in range(40):
            nbytes = sizes_cycle[rep % len(sizes_cycle)]
            off = rep % 3   # unaligned user buffers
            send = [torch.randint(0, 256, (nbytes + off,), generator=g, dtype=torch.uint8).cuda()[off:] for _ in range(n)]
            recv = [torch.full((nbytes + off + 8,), 0xAB, dtype=torch.uint8, device="cuda") for _ in range(n)]
            ranks, peers, sends, bufs, sizes = [], [], [], [], []
            for r in range(n):
                ranks += [r, r]
                peers += [(r + 1) % n, (r - 1) % n]
                sends += [1, 0]
                bufs += [send[r], recv[r][off:off + nbytes]]
                sizes += [nbytes, nbytes]
            k = len(ranks)
            rc = emu_lib.b200EmuP2p(ctx, k, (ctypes.c_int * k)(*ranks), (ctypes.c_int * k)(*peers), (ctypes.c_int * k)(*sends),
                                    _ptrs(bufs), (ctypes.c_size_t * k)(*sizes), 2)
            assert rc == 0, rep
            for r in range(n):
                assert torch.equal(recv[r][off:off + nbytes], send[(r - 1) % n]), "rank %d round %d size %d" % (r, rep, nbytes)
                assert bool((recv[r][:off] == 0xAB).all()) and bool((recv[r][off + nbytes:] == 0xAB).all()), "wrote outside the buffer"
    finally:
        emu_lib.b200EmuDestroy(ctx)
