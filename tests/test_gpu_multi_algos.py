"""Multi-GPU runs of the alternative schedules and of communicator management.

Ring / tree / flagged-line / copy-engine variants are forced with NCCL_ALGO and checked with the
same collective battery as the default selection; then split, one-sided signals, suspend/resume
and pre-multiplied sums.
"""
import pytest

torch = pytest.importorskip("torch")

from mp_util import run_ranks  # noqa: E402
from test_gpu_multi import _check, _colls_rank, _ngpus, _sym_tensor  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("algo", ["Ring", "Tree", "LL", "CE"])
@pytest.mark.parametrize("registered", [True, False])
def test_forced_schedules(algo, registered):
    n = min(_ngpus(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_colls_rank, n, args=(registered, algo), timeout=300)
    _check(res, n)


def test_flagged_lines_with_multicast_stores():
    """The flagged-line all-reduce publishes each line with one multimem.st when asked to."""
    n = min(_ngpus(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_colls_rank, n, args=(True, "LL"), env={"NCCL_B200_LL_MC_MIN_RANKS": "2"}, timeout=300)
    _check(res, n)


@pytest.mark.parametrize("algo", ["NVLS1", "NVLS", "P2P", ""])
def test_barriers_through_multicast(algo):
    """Barrier kernels arrive with one multimem.red on the multicast alias of the flag page; the
    one-shot multimem all-reduce (every rank reads the whole reduced vector) runs on top of it."""
    n = min(_ngpus(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_colls_rank, n, args=(True, algo), env={"NCCL_B200_BARRIER_MC_MIN_RANKS": "2"}, timeout=300)
    _check(res, n)


def test_one_shot_multimem_allreduce_unicast_barrier():
    n = min(_ngpus(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_colls_rank, n, args=(True, "NVLS1"), env={"NCCL_B200_BARRIER_MC_MIN_RANKS": "0"}, timeout=300)
    _check(res, n)


def _back_to_back_rank(rank, nranks, uid, mc):
    """Many small collectives issued without any host synchronisation in between: with programmatic
    dependent launch the next kernel is resident while the previous one drains, so this is where a
    kernel that read an epoch or a buffer too early would show."""
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    n = nranks
    numel = 2048
    x = _sym_tensor(comm, numel, torch.float32)
    y = _sym_tensor(comm, numel, torch.float32)
    g = _sym_tensor(comm, numel * n, torch.float32)
    x.fill_(float(rank + 1))
    torch.cuda.synchronize()
    bad = 0
    for rounds in range(3):
        for i in range(60):
            # y = sum(x) ; x = y / n' chain: every call consumes the previous call's output
            comm.all_reduce(x, y)
            y.mul_(1.0 / n)   # a kernel of the caller between two collectives; keeps the values bounded
            comm.all_gather(y[:numel // n], g[:numel])
            comm.reduce_scatter(g[:numel], x[:numel // n])
            comm.all_reduce(y, x, op="max")
        torch.cuda.synchronize()
        # all ranks must agree bit for bit on x after the chain
        chk = x.clone()
        comm.all_reduce(chk, op="max")
        torch.cuda.synchronize()
        if not torch.equal(chk, x):
            bad += 1
        x.fill_(float(rank + 1))
        torch.cuda.synchronize()
        comm.all_reduce(x, y)   # re-establish the barrier between the refill and the next round
        torch.cuda.synchronize()
    err = comm.async_error()
    comm.destroy()
    return {"bad": bad, "err": err}


@pytest.mark.parametrize("mc", [0, 2])
def test_back_to_back_small_collectives(mc):
    n = min(_ngpus(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_back_to_back_rank, n, args=(mc,), env={"NCCL_B200_BARRIER_MC_MIN_RANKS": str(mc), "NCCL_B200_LL_MC_MIN_RANKS": str(mc)}, timeout=300)
    for r in range(n):
        assert res[r]["bad"] == 0 and res[r]["err"] == 0, res[r]


def test_copy_collectives_on_bulk_engines(tmp_path):
    """A selection table that sends every copy collective to the bulk-copy kernels (push, pull and multicast forms)."""
    import json
    n = min(_ngpus(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    big = 1 << 40
    table = {str(n): {"all_gather": [[big, "BMC", 4]], "all_to_all": [[big, "BPULL", 3]], "broadcast": [[big, "BPUSH", 2]]}}
    path = tmp_path / "bulk_table.json"
    path.write_text(json.dumps(table))
    for registered in (True, False):
        res = run_ranks(_colls_rank, n, args=(registered, ""), env={"NCCL_TUNING_FILE": str(path)}, timeout=300)
        _check(res, n)


def test_broadcast_shared_out_among_the_other_ranks(tmp_path):
    """A selection table that sends every broadcast to the shared-out form: with registered buffers the non-root ranks
    pull from the root's window (found through the descriptor the root publishes inside the kernel); with unregistered
    ones the form does not apply and the default path runs."""
    import json
    n = min(_ngpus(), 8)
    if n < 3:
        pytest.skip("needs at least three GPUs")
    table = {str(n): {"broadcast": [[1 << 40, "SPLIT", 6]]}}
    path = tmp_path / "split_table.json"
    path.write_text(json.dumps(table))
    for registered in (True, False):
        res = run_ranks(_colls_rank, n, args=(registered, ""), env={"NCCL_TUNING_FILE": str(path)}, timeout=300)
        _check(res, n)


@pytest.mark.parametrize("algo", ["", "P2P"])
def test_unregistered_reductions_pipelined_through_small_staging(algo):
    """A 2 MiB staging area and a 1 MiB pipelining threshold: the 4 MiB all-reduce of the battery runs as several
    pieces whose copies overlap the kernels on a side stream."""
    n = min(_ngpus(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    env = {"NCCL_B200_SCRATCH_MB": "2", "NCCL_B200_STAGE_PIPELINE_MIN": "1048576"}
    res = run_ranks(_colls_rank, n, args=(False, algo), env=env, timeout=300)
    _check(res, n)


def _types_rank(rank, nranks, uid, algo):
    """All-reduce and reduce-scatter of every type / operator pair that has a multimem.ld_reduce form
    (plus one without, which must fall back), on registered buffers, checked on the device."""
    import os
    import torch
    os.environ["NCCL_ALGO"] = algo
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    n = nranks
    f8 = [torch.float8_e4m3fn, torch.float8_e5m2] if hasattr(torch, "float8_e4m3fn") else []
    cases = [(torch.float16, "sum"), (torch.float16, "max"), (torch.float16, "min"), (torch.bfloat16, "min"), (torch.float64, "sum"),
             (torch.int64, "sum"), (torch.int64, "max"), (torch.int64, "min"), (torch.int32, "min"), (torch.float32, "max")] + [(t, "sum") for t in f8]
    bad = []
    numel = 8192 * n + 16 * n

    def make(p, dtype):
        g = torch.Generator().manual_seed(500 + p)
        if dtype.is_floating_point:
            return (torch.randn(numel, generator=g).clamp(-2, 2)).to(dtype)
        return torch.randint(-1000, 1000, (numel,), generator=g).to(dtype)

    for dtype, op in cases:
        x = _sym_tensor(comm, numel, dtype)
        y = _sym_tensor(comm, numel, dtype)
        x.copy_(make(rank, dtype))
        comm.all_reduce(x, y, op=op)
        z = _sym_tensor(comm, numel // n, dtype)
        comm.reduce_scatter(x, z, op=op)
        torch.cuda.synchronize()
        ins = [make(p, dtype).cuda() for p in range(n)]
        acc_t = torch.float64 if dtype == torch.float64 else torch.float32 if dtype.is_floating_point else torch.int64
        acc = ins[0].to(acc_t)
        for t in ins[1:]:
            acc = acc + t.to(acc_t) if op == "sum" else torch.maximum(acc, t.to(acc_t)) if op == "max" else torch.minimum(acc, t.to(acc_t))
        if dtype in f8:
            # the switch adds fp8 lanes with an fp16 accumulator: allow one fp8 step plus the accumulator's rounding
            step = 2 ** -3 if dtype == torch.float8_e4m3fn else 2 ** -2
            okf = lambda got, want: bool(((got.float() - want).abs() <= step * want.abs() + 2 ** -5).all())   # noqa: E731
        elif dtype.is_floating_point and op == "sum":
            tol = {torch.float16: 2 ** -9, torch.float64: 1e-12}[dtype]
            okf = lambda got, want: torch.allclose(got.to(acc_t), want, rtol=tol, atol=tol)   # noqa: E731
        else:
            okf = lambda got, want: torch.equal(got.to(acc_t), want)   # noqa: E731
        if not okf(y, acc):
            bad.append(("all_reduce", str(dtype), op))
        per = numel // n
        if not okf(z, acc[rank * per:(rank + 1) * per]):
            bad.append(("reduce_scatter", str(dtype), op))
    err = comm.async_error()
    comm.destroy()
    return {"bad": bad, "err": err}


@pytest.mark.parametrize("algo", ["NVLS", "P2P", "LL"])
def test_reduction_types_on_gpus(algo):
    n = min(_ngpus(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_types_rank, n, args=(algo,), timeout=300)
    for r in range(n):
        assert res[r]["bad"] == [] and res[r]["err"] == 0, res[r]


def _mgmt_rank(rank, nranks, uid):
    import ctypes
    import torch
    torch.cuda.set_device(rank)
    from nccl_b200 import Communicator, _lib
    from nccl_b200.core import FP32
    comm = Communicator(nranks, rank, uid)
    lib = comm.lib
    out = {}
    # split in two halves (odd / even ranks), all-reduce inside each
    sub = comm.split(rank % 2, key=rank)
    x = torch.full((1000,), float(rank + 1), device="cuda")
    sub.all_reduce(x)
    torch.cuda.synchronize()
    out["split_sum"] = float(x[0])
    out["split_size"] = sub.nranks
    sub.destroy()
    # pre-multiplied sum: sum_r (0.5 * x_r)
    op = comm.premul_sum(0.5, FP32)
    y = torch.full((4096,), float(rank + 1), device="cuda")
    z = torch.empty_like(y)
    comm.all_reduce(y, z, op=op)
    torch.cuda.synchronize()
    out["premul"] = float(z[7])
    comm.destroy_op(op)
    # one-sided put + signal around a ring: every rank writes into its successor's window
    win_t = _sym_tensor(comm, 1024, torch.float32)
    win_t.zero_()
    torch.cuda.synchronize()
    win = comm._windows[next(iter(comm._windows))]
    src = torch.full((1024,), 100.0 + rank, device="cuda")
    nxt, prv = (rank + 1) % nranks, (rank - 1) % nranks
    lib.ncclPutSignal.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                                  ctypes.c_int, ctypes.c_int, ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p]

    class Desc(ctypes.Structure):
        _fields_ = [("opCnt", ctypes.c_int), ("peer", ctypes.c_int), ("sigIdx", ctypes.c_int), ("ctx", ctypes.c_int)]
    lib.ncclWaitSignal.argtypes = [ctypes.c_int, ctypes.POINTER(Desc), ctypes.c_void_p, ctypes.c_void_p]
    st = torch.cuda.current_stream().cuda_stream
    # a barrier first: the target must have zeroed its window before anybody writes into it
    b = torch.zeros(1, device="cuda")
    comm.all_reduce(b)
    for _ in range(2):
        _lib.check(lib.ncclPutSignal(src.data_ptr(), 1024, FP32, nxt, win, 0, 3, 0, 0, comm.handle, st), "ncclPutSignal", lib)
        d = Desc(1, prv, 3, 0)
        _lib.check(lib.ncclWaitSignal(1, ctypes.byref(d), comm.handle, st), "ncclWaitSignal", lib)
    torch.cuda.synchronize()
    out["put"] = float(win_t[5])
    # suspend / resume: the resource window goes away and comes back, collectives still work
    before = comm.mem_stats(0)
    comm.suspend()
    out["suspended_flag"] = comm.mem_stats(1)
    out["suspendable_after"] = comm.mem_stats(0)
    comm.resume()
    w = torch.full((1 << 16,), 1.0, device="cuda")
    comm.all_reduce(w)
    torch.cuda.synchronize()
    out["after_resume"] = float(w[0])
    # signals start again from zero with the new resource window: one more put / signal / wait round
    src.fill_(200.0 + rank)
    _lib.check(lib.ncclPutSignal(src.data_ptr(), 1024, FP32, nxt, win, 0, 3, 0, 0, comm.handle, st), "ncclPutSignal", lib)
    d = Desc(1, prv, 3, 0)
    _lib.check(lib.ncclWaitSignal(1, ctypes.byref(d), comm.handle, st), "ncclWaitSignal", lib)
    torch.cuda.synchronize()
    out["put_after_resume"] = float(win_t[5])
    out["suspendable_before"] = before
    assert comm.async_error() == 0
    comm.destroy()
    return out


def test_split_premul_signals_suspend():
    n = min(_ngpus(), 8)
    if n < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_mgmt_rank, n, timeout=300)
    for r in range(n):
        o = res[r]
        members = [q for q in range(n) if q % 2 == r % 2]
        assert o["split_size"] == len(members)
        assert o["split_sum"] == sum(q + 1 for q in members)
        assert o["premul"] == 0.5 * sum(q + 1 for q in range(n))
        assert o["put"] == 100.0 + (r - 1) % n
        assert o["suspended_flag"] == 1 and o["suspendable_after"] == 0 and o["suspendable_before"] > 0
        assert o["after_resume"] == float(n)
        assert o["put_after_resume"] == 200.0 + (r - 1) % n
