"""Runs a function as N rank processes on this host and collects their results.

Ranks are separate interpreter processes (spawn) because the library keeps per-process state
(bootstrap root threads, CUDA contexts). The unique id travels through a multiprocessing pipe,
the way a launcher would broadcast it.
"""
import multiprocessing as mp
import os
import traceback


def _entry(fn, rank, nranks, uid_conn, result_q, env, args):
    try:
        os.environ.update(env)
        import sys
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        uid = uid_conn.recv()
        out = fn(rank, nranks, uid, *args)
        result_q.put((rank, "ok", out))
    except BaseException as e:  # noqa: BLE001 - report every failure to the parent
        result_q.put((rank, "error", "%s\n%s" % (e, traceback.format_exc())))


def run_ranks(fn, nranks, args=(), env=None, timeout=120, make_uid=None, expect_fail=(), may_exit=()):
    """fn(rank, nranks, uid_bytes, *args) runs in nranks processes; returns {rank: result}.
    Ranks listed in may_exit are allowed to leave (os._exit) without reporting a result."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    env = dict(env or {})
    pipes = [ctx.Pipe(duplex=False) for _ in range(nranks)]
    procs = [ctx.Process(target=_entry, args=(fn, r, nranks, pipes[r][0], q, env, args)) for r in range(nranks)]
    for p in procs:
        p.start()
    if make_uid is None:
        from nccl_b200 import get_unique_id
        uid = get_unique_id()
    else:
        uid = make_uid()
    for r in range(nranks):
        pipes[r][1].send(uid)
    results = {}
    try:
        for _ in range(nranks - len(may_exit)):
            rank, status, out = q.get(timeout=timeout)
            if status != "ok" and rank not in expect_fail:
                raise AssertionError("rank %d failed: %s" % (rank, out))
            results[rank] = out if status == "ok" else ("error", out)
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    return results
