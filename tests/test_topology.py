"""Topology XML -> system graph -> paths -> channel search -> analytic model, on injected files
(the way NCCL_TOPO_FILE lets a machine be described without owning it). CPU only."""
import ctypes
import json
import os

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def analyze(lib):
    lib.b200TopoAnalyze.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]

    def run(name):
        text = open(os.path.join(HERE, "data", name)).read().encode()
        buf = ctypes.create_string_buffer(4096)
        rc = lib.b200TopoAnalyze(text, buf, 4096)
        out = json.loads(buf.value.decode())
        out["rc"] = rc
        return out
    return run


def test_hgx_b200(analyze):
    r = analyze("hgx_b200_8gpu.xml")
    assert r["rc"] == 0 and r["gpus"] == 8 and r["nvswitch"] == 1 and r["nets"] == 8
    assert r["best_path"] == "NVL" and r["worst_path"] == "NVL"
    # 18 links x 40.1 GB/s per GPU: 8 channels at the top of the sm_100 speed ladder (90 GB/s)
    assert r["speed"] == 90.0 and r["channels"] == 8 and r["type"] == "NVL"
    assert sorted(r["ring0"]) == list(range(8))
    assert abs(r["max_bw"] - 18 * 40.1) < 1.0
    # in-switch reduction beats the ring at 1 MiB in the model, trees win tiny messages
    assert 0 < r["t_nvls_1M"] and 0 < r["t_ring_simple_1M"]
    assert r["t_tree_ll_1K"] < r["t_ring_simple_1M"]


def test_hgx_h100(analyze):
    r = analyze("hgx_h100_8gpu.xml")
    assert r["gpus"] == 8 and r["type"] == "NVL"
    assert r["speed"] <= 60.0 and r["channels"] * r["speed"] <= 18 * 20.6 + 1


def test_pcie_only(analyze):
    r = analyze("pcie_4gpu.xml")
    assert r["gpus"] == 4 and r["nvswitch"] == 0
    assert r["best_path"] == "PIX" and r["worst_path"] == "SYS"
    assert r["channels"] >= 1 and sorted(r["ring0"]) == [0, 1, 2, 3]
    # GPUs under one switch stay adjacent in the ring: only two hops cross the CPU interconnect
    ring = r["ring0"]
    crossings = sum(1 for i in range(4) if (ring[i] // 2) != (ring[(i + 1) % 4] // 2))
    assert crossings == 2


def test_nvlink_mesh(analyze):
    r = analyze("nvlink_mesh_4gpu.xml")
    assert r["gpus"] == 4 and r["best_path"] == "NVL" and r["worst_path"] == "NVL" and r["type"] == "NVL"
    # 4 links x 20.6 GB/s between each pair; rings use two of a GPU's three neighbours
    assert r["channels"] * r["speed"] >= 80


def test_malformed_xml(lib):
    lib.b200TopoAnalyze.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]
    buf = ctypes.create_string_buffer(1024)
    assert lib.b200TopoAnalyze(b"<system><cpu numaid='0'></system>", buf, 1024) == 1
    assert lib.b200TopoAnalyze(b"<nope/>", buf, 1024) == 2


def test_binary_trees(lib):
    lib.b200Btree.argtypes = [ctypes.c_int, ctypes.c_int] + [ctypes.POINTER(ctypes.c_int)] * 3
    lib.b200Dtree.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
    for n in range(1, 34):
        parents, children = {}, {}
        for r in range(n):
            u, d0, d1 = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
            lib.b200Btree(n, r, ctypes.byref(u), ctypes.byref(d0), ctypes.byref(d1))
            parents[r] = u.value
            children[r] = [c for c in (d0.value, d1.value) if c >= 0]
        # one root, everybody reachable, parent/child views agree
        assert sum(1 for r in range(n) if parents[r] == -1) == 1
        for r in range(n):
            for c in children[r]:
                assert 0 <= c < n and parents[c] == r
        seen, stack = set(), [next(r for r in range(n) if parents[r] == -1)]
        while stack:
            x = stack.pop()
            seen.add(x)
            stack += children[x]
        assert len(seen) == n
        # double tree: every rank is interior in at most one of the two trees (n > 2)
        if n > 2:
            interior0 = {r for r in range(n) if children[r]}
            interior1 = set()
            for r in range(n):
                o = (ctypes.c_int * 6)()
                lib.b200Dtree(n, r, o)
                if o[4] >= 0 or o[5] >= 0:
                    interior1.add(r)
            assert len(interior0 & interior1) <= 1, (n, interior0 & interior1)


def test_builtin_selection_table_parses(lib):
    """The measured selection table compiled into the library: five collectives for each of 2 to 8 ranks."""
    assert lib.b200TuningDefaultsCheck() == 5 * 7
