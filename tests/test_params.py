"""Parameter registry: environment variables, configuration files and their precedence, the query
API and the ncclparam tool. Each case runs in a child process because parameters are cached."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOOL = os.path.join(ROOT, "nccl_b200", "bin", "ncclparam")


def _child(code, env):
    e = dict(os.environ)
    e.update(env)
    e["PYTHONPATH"] = ROOT
    out = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], env=e, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    return out.stdout


QUERY = """
import ctypes
from nccl_b200 import _lib
lib = _lib.load()
h = ctypes.c_void_p()
lib.ncclParamBind.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]
lib.ncclParamGetI64.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)]
for key in (b"NCCL_B200_NET_SLICE_KB", b"NCCL_RAS_ENABLE"):
    assert lib.ncclParamBind(ctypes.byref(h), key) == 0, key
    v = ctypes.c_int64()
    assert lib.ncclParamGetI64(h, ctypes.byref(v)) == 0
    print(key.decode(), v.value)
assert lib.ncclParamBind(ctypes.byref(h), b"NCCL_NO_SUCH_PARAMETER") != 0
"""


def test_defaults_env_and_conf_precedence(tmp_path):
    out = _child(QUERY, {})
    assert "NCCL_B200_NET_SLICE_KB 512" in out and "NCCL_RAS_ENABLE 1" in out
    conf = tmp_path / "nccl.conf"
    conf.write_text("# comment\nNCCL_B200_NET_SLICE_KB = 128\nNCCL_RAS_ENABLE=0\n")
    out = _child(QUERY, {"NCCL_CONF_FILE": str(conf)})
    assert "NCCL_B200_NET_SLICE_KB 128" in out and "NCCL_RAS_ENABLE 0" in out
    # the process environment wins over the file
    out = _child(QUERY, {"NCCL_CONF_FILE": str(conf), "NCCL_B200_NET_SLICE_KB": "64"})
    assert "NCCL_B200_NET_SLICE_KB 64" in out and "NCCL_RAS_ENABLE 0" in out


def test_key_table_and_tool():
    code = """
    import ctypes
    from nccl_b200 import _lib
    lib = _lib.load()
    table = ctypes.POINTER(ctypes.c_char_p)()
    n = ctypes.c_int()
    lib.ncclParamGetAllParameterKeys.argtypes = [ctypes.POINTER(ctypes.POINTER(ctypes.c_char_p)), ctypes.POINTER(ctypes.c_int)]
    assert lib.ncclParamGetAllParameterKeys(ctypes.byref(table), ctypes.byref(n)) == 0
    keys = [table[i].decode() for i in range(n.value)]
    print(len(keys))
    print("\\n".join(keys))
    """
    out = _child(code, {}).splitlines()
    assert int(out[0]) >= 30
    assert "NCCL_B200_WAIT_TIMEOUT_MS" in out and "NCCL_SOCKET_RETRY_CNT" in out
    tool = subprocess.run([TOOL], capture_output=True, text=True, timeout=60, env=dict(os.environ, NCCL_B200_NET_INFLIGHT="5"))
    assert tool.returncode == 0
    assert "NCCL_B200_NET_INFLIGHT" in tool.stdout and "5" in tool.stdout


TYPED = """
import ctypes
from nccl_b200 import _lib
lib = _lib.load()
h = ctypes.c_void_p()
lib.ncclParamBind.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]
assert lib.ncclParamBind(ctypes.byref(h), b"NCCL_B200_NET_INFLIGHT") == 0
for name, ct in (("I8", ctypes.c_int8), ("I16", ctypes.c_int16), ("I32", ctypes.c_int32), ("I64", ctypes.c_int64),
                 ("U8", ctypes.c_uint8), ("U16", ctypes.c_uint16), ("U32", ctypes.c_uint32), ("U64", ctypes.c_uint64)):
    fn = getattr(lib, "ncclParamGet" + name)
    fn.argtypes = [ctypes.c_void_p, ctypes.POINTER(ct)]
    v = ct()
    assert fn(h, ctypes.byref(v)) == 0, name
    assert v.value == 5, (name, v.value)
assert lib.ncclParamBind(ctypes.byref(h), b"NCCL_SOCKET_IFNAME") == 0
lib.ncclParamGetStr.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_char_p)]
s = ctypes.c_char_p()
assert lib.ncclParamGetStr(h, ctypes.byref(s)) == 0 and s.value == b"lo"
buf = ctypes.create_string_buffer(16)
n = ctypes.c_int()
lib.ncclParamGet.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
assert lib.ncclParamGet(h, buf, 16, ctypes.byref(n)) == 0
print("raw", n.value, buf.raw[:max(n.value, 0)])
"""


def test_typed_getters():
    out = _child(TYPED, {"NCCL_B200_NET_INFLIGHT": "5", "NCCL_SOCKET_IFNAME": "lo"})
    assert out.startswith("raw")


RELOAD = """
import os, sys
from nccl_b200 import _lib, Communicator, get_unique_id
lib = _lib.load()
path = sys.argv[1] if len(sys.argv) > 1 else os.environ["LOG_PATH"]
c = Communicator(1, 0, get_unique_id())      # logging is off: nothing is written
c.destroy()
os.environ["NCCL_DEBUG"] = "INFO"
os.environ["NCCL_DEBUG_FILE"] = path
lib.ncclResetDebugInit()                      # re-reads the logging variables
c = Communicator(1, 0, get_unique_id())
c.destroy()
print(os.path.exists(path) and "Init COMPLETE" in open(path).read())
"""


def test_reset_debug_init_rereads_the_environment(tmp_path):
    out = _child(RELOAD, {"LOG_PATH": str(tmp_path / "log.txt"), "NCCL_B200_HOST_ONLY": "1", "NCCL_DEBUG": ""})
    assert out.strip().endswith("True"), out


WARN_ONCE = """
import ctypes
from nccl_b200 import _lib
lib = _lib.load()
w = ctypes.c_void_p()
lib.ncclCommWindowRegister(None, None, 0, ctypes.byref(w), 0)   # invalid communicator: one WARN line
"""


def _warn_line(env):
    e = {"NCCL_DEBUG": "WARN"}
    e.update(env)
    lines = [l for l in _child(WARN_ONCE, e).splitlines() if "NCCL WARN" in l]
    assert len(lines) == 1, lines
    return lines[0]


def test_time_stamps_of_log_lines():
    import re
    # warnings carry a time stamp by default: local time, seconds
    assert re.match(r"^\[\d{4}-\d\d-\d\d \d\d:\d\d:\d\d\] \S+:\d+:\d+ ", _warn_line({}))
    # none at all
    assert not _warn_line({"NCCL_DEBUG_TIMESTAMP_LEVELS": ""}).startswith("[")
    assert not _warn_line({"NCCL_DEBUG_TIMESTAMP_LEVELS": "^WARN"}).startswith("[")
    assert not _warn_line({"NCCL_DEBUG_TIMESTAMP_FORMAT": ""}).startswith("[")
    assert _warn_line({"NCCL_DEBUG_TIMESTAMP_LEVELS": "INFO,WARN"}).startswith("[")
    # own format: fraction of the second with %Nf, underscores become spaces
    assert re.match(r"^<\d\d:\d\d:\d\d\.\d{3}> \S+:\d+", _warn_line({"NCCL_DEBUG_TIMESTAMP_FORMAT": "<%H:%M:%S.%3f>_"}))
    assert re.match(r"^\d{9}\|", _warn_line({"NCCL_DEBUG_TIMESTAMP_FORMAT": "%9f|"}))


def test_reference_variables_without_a_counterpart_are_listed():
    out = subprocess.run([TOOL, "--all"], capture_output=True, text=True, timeout=60).stdout
    for name in ("NCCL_IB_DISABLE", "NCCL_MNNVL_ENABLE", "NCCL_BUFFSIZE", "NCCL_MEM_SYNC_DOMAIN", "NCCL_CTA_POLICY", "NCCL_WIN_ENABLE",
                 "NCCL_MAX_NCHANNELS", "NCCL_SET_THREAD_NAME", "NCCL_DEBUG_TIMESTAMP_FORMAT", "NCCL_CROSS_NIC", "NCCL_P2P_LEVEL", "NCCL_GIN_TYPE"):
        assert name in out, name


def test_cpu_list_parser_of_the_proxy_affinity():
    """Lists in the form of the kernel's local_cpulist files: ranges, single CPUs, separators, malformed tails."""
    import ctypes
    from nccl_b200 import _lib
    lib = _lib.load()
    out = (ctypes.c_int * 64)()

    def parse(text, cap=64):
        n = lib.b200ParseCpuList(text, out, cap)
        return list(out[:n])

    assert parse(b"0-3,8-9\n") == [0, 1, 2, 3, 8, 9]
    assert parse(b"5") == [5] and parse(b"") == [] and parse(b"2-1") == []
    assert parse(b"0-2, 7") == [0, 1, 2, 7]
    assert parse(b"0-63,64-127", cap=4) == [0, 1, 2, 3]
    assert parse(b"3,x") == [3]


def test_environment_reference_lists_every_registered_parameter():
    """docs/env.md is generated from the registry (python docs/gen_env.py): every variable that `ncclparam --all` prints has its row."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([os.path.join(root, "nccl_b200", "bin", "ncclparam"), "--all"], capture_output=True, text=True, check=True).stdout
    names = [line.split("=", 1)[0].strip() for line in out.splitlines() if "=" in line and "#" in line]
    doc = open(os.path.join(root, "docs", "env.md")).read()
    missing = [n for n in names if "`%s`" % n not in doc]
    assert len(names) > 80 and not missing, missing
