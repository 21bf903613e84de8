"""Multi-node NVLink detection: fabric identity through a fake NVML, cliques from gathered records, environment overrides.
Nothing here touches a GPU; the memory-handle side needs an NVLink fabric that spans hosts."""
import ctypes
import os
import subprocess
import sys

from nccl_b200 import _lib

COMPLETED, IN_PROGRESS = 3, 2


class FabricInfo(ctypes.Structure):
    _fields_ = [("uuid", ctypes.c_uint8 * 16), ("clique", ctypes.c_uint32), ("state", ctypes.c_int32), ("health", ctypes.c_uint32), ("status", ctypes.c_int32)]


def _info(uuid_byte, clique, state=COMPLETED):
    fi = FabricInfo()
    for i in range(16):
        fi.uuid[i] = uuid_byte
    fi.clique, fi.state = clique, state
    return fi


def _clique(infos, me):
    lib = _lib.load()
    arr = (FabricInfo * len(infos))(*infos)
    ranks = (ctypes.c_int * len(infos))()
    dom = ctypes.c_int(0)
    lib.b200MnnvlClique.restype = ctypes.c_int
    n = lib.b200MnnvlClique(arr, len(infos), me, ranks, ctypes.byref(dom))
    return list(ranks[:n]), dom.value


def test_ranks_of_one_clique_form_one_domain():
    infos = [_info(7, 1) for _ in range(8)]
    for me in (0, 5):
        ranks, dom = _clique(infos, me)
        assert ranks == list(range(8)) and dom == 8


def test_two_cliques_in_one_fabric_and_a_foreign_fabric():
    infos = [_info(7, 1), _info(7, 2), _info(7, 1), _info(9, 1), _info(7, 2), _info(7, 1)]
    assert _clique(infos, 0) == ([0, 2, 5], 5)
    assert _clique(infos, 1) == ([1, 4], 5)
    # rank 3 is alone in its fabric: no multi-rank domain for it
    assert _clique(infos, 3)[0] == []


def test_fabric_not_ready_or_without_uuid_means_no_clique():
    infos = [_info(7, 1), _info(7, 1, IN_PROGRESS)]
    assert _clique(infos, 0)[0] == []
    infos = [_info(0, 1), _info(0, 1)]
    assert _clique(infos, 0)[0] == []


_FAKE = r'''
import ctypes, os, sys
sys.path.insert(0, os.environ["REPO"])
from nccl_b200 import _lib
lib = _lib.load()

class Info(ctypes.Structure):
    _fields_ = [("version", ctypes.c_uint), ("uuid", ctypes.c_ubyte * 16), ("status", ctypes.c_int), ("clique", ctypes.c_uint),
                ("state", ctypes.c_ubyte), ("health", ctypes.c_uint)]

seen = {}
BY_BUS = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p))
FABRIC = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(Info))

def by_bus(bus, out):
    seen["bus"] = bus.decode()
    out[0] = 0x1234
    return 0

def fabric(dev, info):
    seen["version"] = info[0].version
    for i in range(16):
        info[0].uuid[i] = 0xA0 + i
    info[0].clique, info[0].state, info[0].health = 42, 3, 0x11
    return 0

class Api(ctypes.Structure):   # the table of entry points, in the order of the library's NVML wrapper
    _fields_ = [("count", ctypes.c_void_p), ("by_index", ctypes.c_void_p), ("by_bus", BY_BUS), ("index", ctypes.c_void_p), ("nvl_state", ctypes.c_void_p),
                ("nvl_remote", ctypes.c_void_p), ("p2p", ctypes.c_void_p), ("cc", ctypes.c_void_p), ("fabric", FABRIC)]

api = Api(None, None, BY_BUS(by_bus), None, None, None, None, None, FABRIC(fabric))
lib.b200NvmlSetApiForTest(ctypes.byref(api))

class FabricInfo(ctypes.Structure):
    _fields_ = [("uuid", ctypes.c_uint8 * 16), ("clique", ctypes.c_uint32), ("state", ctypes.c_int32), ("health", ctypes.c_uint32), ("status", ctypes.c_int32)]

fi = FabricInfo()
lib.b200FabricInfoQuery(b"0000:1b:00.0", ctypes.byref(fi))
lib.b200NvmlSetApiForTest(None)
print(seen["bus"], seen["version"] >> 24, seen["version"] & 0xFFFFFF, bytes(fi.uuid).hex(), fi.clique, fi.state, fi.health)
'''


def _run_fake(extra_env):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, REPO=root, **extra_env)
    out = subprocess.run([sys.executable, "-c", _FAKE], env=env, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    return out.stdout.split()


def test_fabric_identity_comes_from_nvml():
    bus, ver, size, uuid, clique, state, health = _run_fake({})
    assert bus == "0000:1b:00.0" and ver == "2" and int(size) == 36
    assert uuid == bytes(range(0xA0, 0xB0)).hex() and (clique, state, health) == ("42", "3", "17")


def test_environment_replaces_uuid_and_clique():
    _, _, _, uuid, clique, _, _ = _run_fake({"NCCL_MNNVL_UUID": "0x1122334455667788", "NCCL_MNNVL_CLIQUE_ID": "5"})
    half = (0x1122334455667788).to_bytes(8, "little").hex()
    assert uuid == half + half and clique == "5"
