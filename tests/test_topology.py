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


def _graphs(lib, name, inter=0, cross_nic=0):
    import re
    lib.b200TopoGraphs.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
    buf = ctypes.create_string_buffer(1 << 18)
    text = open(os.path.join(HERE, "data", name)).read().encode()
    assert lib.b200TopoGraphs(text, inter, cross_nic, buf, 1 << 18) == 0
    xml = buf.value.decode()
    out = {}
    for m in re.finditer(r'<graph id="(\d)"([^>]*?)/?>(.*?)(?=<graph |</graphs>)', xml, re.S):
        attrs = dict(re.findall(r'(\w+)="([^"]*)"', m.group(2)))
        chans = [[(k, int(v)) for k, v in re.findall(r'<(net|gpu) dev="(\d+)"', ch)] for ch in re.findall(r"<channel>(.*?)</channel>", m.group(3), re.S)]
        out[int(m.group(1))] = (attrs, chans)
    return xml, out


def test_tree_and_nvls_graphs_inside_one_node(lib):
    _, g = _graphs(lib, "hgx_b200_8gpu.xml")
    ring, tree, nvls = g[0], g[1], g[2]
    assert ring[0]["pattern"] == "4" and int(ring[0]["nchannels"]) == 8 and float(ring[0]["speedintra"]) == 90.0
    # tree links carry traffic in both directions, so fewer chains fit than rings
    assert tree[0]["pattern"] == "1" and 1 <= int(tree[0]["nchannels"]) <= 8
    for attrs, chans in (ring, tree, nvls):
        assert len(chans) == int(attrs["nchannels"])
        for ch in chans:
            assert all(k == "gpu" for k, _ in ch) and sorted(v for _, v in ch) == list(range(8))
    # NVLS: one head per GPU, 8 x 90 GB/s fills the 18 links of every GPU
    assert nvls[0]["pattern"] == "5" and int(nvls[0]["nchannels"]) == 8 and float(nvls[0]["speedintra"]) == 90.0
    assert sorted(ch[0][1] for ch in nvls[1]) == list(range(8))
    # no switch, no NVLS graph
    _, g = _graphs(lib, "pcie_4gpu.xml")
    assert int(g[2][0]["nchannels"]) == 0 and int(g[1][0]["nchannels"]) >= 1


def test_channels_attach_to_the_closest_nic_across_nodes(lib):
    _, g = _graphs(lib, "hgx_b200_8gpu.xml", inter=1)
    ring, tree = g[0], g[1]
    assert ring[0]["typeinter"] == "PIX" and ring[0]["typeintra"] == "NVL"
    # a 400 Gb/s NIC carries 50 GB/s: the per-NIC sum of channel speeds stays below it
    per_nic = {}
    for ch in ring[1]:
        assert ch[0][0] == "net" and ch[-1][0] == "net" and sorted(v for k, v in ch if k == "gpu") == list(range(8))
        # in this machine NIC i hangs off the PCI switch of GPU i: the ring enters at that GPU and leaves through the same NIC
        assert ch[1] == ("gpu", ch[0][1]) and ch[-1][1] == ch[0][1]
        per_nic[ch[0][1]] = per_nic.get(ch[0][1], 0) + float(ring[0]["speedinter"])
    assert len(per_nic) == 8 and max(per_nic.values()) <= 50.0
    # balanced tree: the network traffic of a chain is spread over its first two GPUs, each through its own NIC
    for ch in tree[1]:
        gpus = [v for k, v in ch if k == "gpu"]
        assert ch[0] == ("net", gpus[0]) and ch[-1] == ("net", gpus[1])


def test_graph_file_round_trip_and_refusals(lib):
    lib.b200TopoGraphReload.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
    for name, inter, n in (("hgx_b200_8gpu.xml", 0, 8), ("hgx_b200_8gpu.xml", 1, 8), ("pcie_4gpu.xml", 0, 4)):
        xml, _ = _graphs(lib, name, inter)
        buf = ctypes.create_string_buffer(1 << 18)
        assert lib.b200TopoGraphReload(xml.encode(), n, buf, 1 << 18) == 0
        assert buf.value.decode() == xml
    xml, _ = _graphs(lib, "pcie_4gpu.xml")
    buf = ctypes.create_string_buffer(1 << 16)
    # a channel that visits a GPU twice
    bad = xml.replace('<gpu dev="1"/>', '<gpu dev="0"/>', 1)
    assert lib.b200TopoGraphReload(bad.encode(), 4, buf, 1 << 16) == 10 and b"exactly once" in buf.value
    # a channel count that disagrees with the channels
    bad = xml.replace('nchannels="4"', 'nchannels="3"', 1)
    assert lib.b200TopoGraphReload(bad.encode(), 4, buf, 1 << 16) == 10 and b"nchannels" in buf.value
    # a file written for another number of ranks
    assert lib.b200TopoGraphReload(xml.encode(), 8, buf, 1 << 16) == 10
