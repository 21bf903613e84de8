"""From sweep results to a selection table and back into the library's parser. CPU only."""
import ctypes
import json

from nccl_b200.utils import tune

FUNC_BROADCAST, FUNC_ALLGATHER, FUNC_ALLREDUCE = 0, 2, 4
ALGO_LL, ALGO_P2P, ALGO_NVLS, ALGO_CE, ALGO_NVLS1 = 1, 2, 3, None, 8
MODE_PUSH, MODE_PULL, MODE_MC, MODE_SPLIT, MODE_BULK = 0, 1, 2, 3, 4


def _cell(times):
    best = min(times, key=times.get)
    return {"best": best, "time_us": times[best], "busbw_GBps": 0.0, "all": times}


def test_rows_prefer_few_ctas_copy_engines_and_merge_runs():
    res = {
        "1024": _cell({"LL": 5.0, "LL+mc": 4.0, "PUSH/2": 9.0}),
        "4096": _cell({"LL": 5.5, "LL+mc": 4.4, "PUSH/2": 9.5}),
        # 8 CTAs are within 3 % of 32: the smaller count wins
        "1048576": _cell({"PUSH/8": 20.3, "PUSH/32": 20.0, "PUSH/32+mb": 25.0, "BPUSH/8": 22.0}),
        # the copy engines tie with the best kernel: no SM at all
        "268435456": _cell({"PUSH/128": 400.0, "CE": 405.0, "BMC/16": 420.0}),
    }
    rows = tune.rows_from(res, use_mc=True, use_mb=False)
    assert [r[1:] for r in rows] == [["LL", 0], ["PUSH", 8], ["CE", 0]]
    assert rows[0][0] == int((4096 * 1048576) ** 0.5) and rows[-1][0] == 1 << 40   # limits between neighbouring sizes
    # with the barrier switch on, the "+mb" twin is what counts where one was measured
    rows_mb = tune.rows_from(res, use_mc=False, use_mb=True)
    assert rows_mb[1][1:] == ["PUSH", 8] and rows_mb[0][1:] == ["LL", 0]


def test_switches_are_decided_from_the_geometric_mean():
    res = {"all_reduce": {"8": _cell({"LL": 6.0, "LL+mc": 5.0}), "1048576": _cell({"NVLS/8": 20.0, "NVLS/8+mb": 20.1})}}
    mc, mb = tune.decide_toggles(res)
    assert mc and not mb


def test_every_variant_name_is_understood_by_the_library(lib):
    lib.b200TuningLookup.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_ulonglong, ctypes.c_char_p, ctypes.c_int]
    table = {"4": {"all_reduce": [[1000, "LL", 0], [2000, "NVLS1", 8], [3000, "NVLS", 4], [1 << 40, "P2P", 64]],
                   "all_gather": [[1000, "PUSH", 2], [2000, "PULL", 4], [3000, "MC", 8], [4000, "BPUSH", 16], [5000, "BPULL", 16], [6000, "BMC", 8], [1 << 40, "CE", 0]],
                   "broadcast": [[1 << 40, "SPLIT", 12]]},
             "llMcMin": 4, "barrierMcMin": 0}
    text = json.dumps(table).encode()

    def pick(func, nbytes):
        buf = ctypes.create_string_buffer(64)
        assert lib.b200TuningLookup(text, func, 4, nbytes, buf, 64) == 0
        return [int(x) for x in buf.value.split()]

    assert pick(FUNC_ALLREDUCE, 500)[0] == ALGO_LL and pick(FUNC_ALLREDUCE, 1500) == [ALGO_NVLS1, -1, 8]
    assert pick(FUNC_ALLREDUCE, 2500) == [ALGO_NVLS, -1, 4] and pick(FUNC_ALLREDUCE, 1 << 30) == [ALGO_P2P, -1, 64]
    assert [pick(FUNC_ALLGATHER, b)[1] for b in (500, 1500, 2500, 3500, 4500, 5500)] == [MODE_PUSH, MODE_PULL, MODE_MC, MODE_PUSH | MODE_BULK, MODE_PULL | MODE_BULK, MODE_MC | MODE_BULK]
    assert pick(FUNC_ALLGATHER, 1 << 30)[2] == 0
    assert pick(FUNC_BROADCAST, 1 << 20)[1:] == [MODE_SPLIT, 12]
    buf = ctypes.create_string_buffer(64)
    assert lib.b200TuningLookup(b'{"4": {"all_reduce": [[1000, "LL"]]}}', FUNC_ALLREDUCE, 4, 10, buf, 64) == 1   # malformed row
    assert lib.b200TuningLookup(text, FUNC_ALLREDUCE, 7, 10, buf, 64) == 2                                        # no rows for 7 ranks
