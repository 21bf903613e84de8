"""Host-memory communicators: TCP bootstrap + ring reduce-scatter/all-gather executed on the CPU."""
import numpy as np
import pytest

from mp_util import run_ranks


def _allreduce_rank(rank, nranks, uid, count):
    import numpy as np
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    rng = np.random.default_rng(1000 + rank)
    x = rng.standard_normal(count).astype(np.float32)
    y = np.empty_like(x)
    comm.all_reduce(x, y, op="sum")
    comm.destroy()
    return y


def test_allreduce_sum_two_ranks_1mi_fp32():
    # 2 processes, 1,048,576 fp32 values from N(0,1) with seed 1000+rank, exact check against the host sum
    count = 1 << 20
    res = run_ranks(_allreduce_rank, 2, args=(count,))
    a = np.random.default_rng(1000).standard_normal(count).astype(np.float32)
    b = np.random.default_rng(1001).standard_normal(count).astype(np.float32)
    expect = a + b
    assert np.array_equal(res[0], expect)
    assert np.array_equal(res[1], expect)


def _all_colls_rank(rank, nranks, uid):
    import numpy as np
    from nccl_b200 import Communicator, group
    comm = Communicator(nranks, rank, uid)
    n = nranks
    out = {}
    x = (np.arange(1000, dtype=np.float64) + rank)
    y = np.empty_like(x)
    comm.all_reduce(x, y, op="max")
    out["ar_max"] = y.copy()
    comm.all_reduce(x, y, op="avg")
    out["ar_avg"] = y.copy()
    g = np.empty(n * 10, dtype=np.int32)
    comm.all_gather(np.full(10, rank, dtype=np.int32), g)
    out["ag"] = g
    rs = np.empty(7, dtype=np.int64)
    comm.reduce_scatter(np.arange(7 * n, dtype=np.int64) * (rank + 1), rs)
    out["rs"] = rs
    b = np.arange(33, dtype=np.float32) if rank == 1 else np.zeros(33, dtype=np.float32)
    comm.broadcast(b, b, root=1)
    out["bc"] = b
    r = np.zeros(5, dtype=np.float32)
    comm.reduce(np.full(5, rank + 1, dtype=np.float32), r, root=0, op="prod")
    out["red"] = r
    a2a = np.empty(n * 3, dtype=np.int32)
    comm.all_to_all(np.repeat(np.arange(n, dtype=np.int32) + 100 * rank, 3), a2a)
    out["a2a"] = a2a
    # ring send/recv in a group
    nxt, prv = (rank + 1) % n, (rank - 1) % n
    rb = np.empty(4, dtype=np.float32)
    with group():
        comm.send(np.full(4, rank, dtype=np.float32), nxt)
        comm.recv(rb, prv)
    out["ring"] = rb
    half = np.full(6, np.float16(1.5) * (rank + 1), dtype=np.float16)
    hout = np.empty_like(half)
    comm.all_reduce(half, hout)
    out["half"] = hout
    comm.destroy()
    return out


@pytest.mark.parametrize("nranks", [2, 3, 4])
def test_every_collective_on_host(nranks):
    res = run_ranks(_all_colls_rank, nranks)
    n = nranks
    base = np.arange(1000, dtype=np.float64)
    for r in range(n):
        o = res[r]
        assert np.array_equal(o["ar_max"], base + n - 1)
        assert np.allclose(o["ar_avg"], base + (n - 1) / 2)
        assert np.array_equal(o["ag"], np.repeat(np.arange(n, dtype=np.int32), 10))
        tot = sum(range(1, n + 1))
        assert np.array_equal(o["rs"], np.arange(7 * n, dtype=np.int64)[7 * r:7 * r + 7] * tot)
        assert np.array_equal(o["bc"], np.arange(33, dtype=np.float32))
        if r == 0:
            assert np.array_equal(o["red"], np.full(5, float(np.prod(np.arange(1, n + 1))), dtype=np.float32))
        assert np.array_equal(o["a2a"], np.repeat(np.arange(n, dtype=np.int32) * 100 + r, 3))
        assert np.array_equal(o["ring"], np.full(4, (r - 1) % n, dtype=np.float32))
        assert np.array_equal(o["half"], np.full(6, 1.5 * tot, dtype=np.float16))


def _logstep_rank(rank, nranks, uid, count):
    import numpy as np
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    n = nranks
    rng = np.random.default_rng(7 + rank)
    mine = rng.integers(-1000, 1000, size=count).astype(np.int64)
    gathered = np.empty(count * n, dtype=np.int64)
    comm.all_gather(mine, gathered)
    full = rng.integers(-1000, 1000, size=count * n).astype(np.int64)
    part = np.empty(count, dtype=np.int64)
    comm.reduce_scatter(full, part, op="sum")
    favg = np.full(count * n, float(rank + 1), dtype=np.float32)
    pavg = np.empty(count, dtype=np.float32)
    comm.reduce_scatter(favg, pavg, op="avg")
    comm.destroy()
    return gathered, part, pavg


@pytest.mark.parametrize("algo", ["PAT", "Ring", None])
@pytest.mark.parametrize("nranks", [3, 5, 8])
def test_log_step_all_gather_and_reduce_scatter(nranks, algo):
    """The log-step (PAT-style) schedule gives the results of the ring schedule for every rank count, power of two or not."""
    count = 3001
    env = {"NCCL_ALGO": algo} if algo else {}
    res = run_ranks(_logstep_rank, nranks, args=(count,), env=env, timeout=200)
    n = nranks
    mines, fulls = [], []
    for r in range(n):
        rng = np.random.default_rng(7 + r)
        mines.append(rng.integers(-1000, 1000, size=count).astype(np.int64))
        fulls.append(rng.integers(-1000, 1000, size=count * n).astype(np.int64))
    total = sum(fulls)
    for r in range(n):
        g, p, a = res[r]
        assert np.array_equal(g, np.concatenate(mines))
        assert np.array_equal(p, total[r * count:(r + 1) * count])
        assert np.allclose(a, (n + 1) / 2.0)


def _bcast_rank(rank, nranks, uid):
    import numpy as np
    from nccl_b200 import Communicator
    comm = Communicator(nranks, rank, uid)
    out = []
    for root in range(nranks):
        buf = np.arange(5000, dtype=np.float32) + 100 * root if rank == root else np.zeros(5000, dtype=np.float32)
        res = np.empty_like(buf)
        comm.broadcast(buf, res, root)
        out.append(res.copy())
    comm.destroy()
    return out


@pytest.mark.parametrize("nranks", [2, 5, 8])
def test_broadcast_from_every_root(nranks):
    """The binomial-tree broadcast of the host plane delivers the root's data for every root and rank count."""
    res = run_ranks(_bcast_rank, nranks, timeout=200)
    for r in range(nranks):
        for root in range(nranks):
            assert np.array_equal(res[r][root], np.arange(5000, dtype=np.float32) + 100 * root)
