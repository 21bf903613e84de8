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
