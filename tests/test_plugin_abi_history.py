"""Plugins written against earlier interface versions, and the reference's own example plugins.

Deployed plugins export tables older than the newest one: the net backend of the examples is built
here behind interfaces v8 to v11 (one table per library) and must carry host traffic through the
library's adapters; small tuner plugins speaking v2, v3 and v4 must be consulted. When the reference
tree is present, its example net, tuner and profiler plugins are compiled unchanged and loaded.
"""
import os
import shutil
import subprocess

import pytest

from mp_util import run_ranks
from test_plugins import BASE, ROOT, _check, _rank

# the reference tree, when it is checked out next to this repository (or named by NCCL_REFERENCE_DIR)
REF = os.path.join(os.environ.get("NCCL_REFERENCE_DIR", os.path.join(os.path.dirname(ROOT), "reference")), "plugins")
CUDA_INC = "/usr/local/cuda/include"

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs a C++ compiler")


def _logs(tmp_path):
    return "".join(open(os.path.join(tmp_path, p)).read() for p in os.listdir(tmp_path) if p.startswith("log."))


@pytest.mark.parametrize("abi", [8, 9, 10, 11])
def test_net_plugin_of_an_earlier_interface(tmp_path, abi):
    so = str(tmp_path / ("libunix_v%d.so" % abi))
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-I" + os.path.join(ROOT, "include"), "-I" + CUDA_INC,
                           "-DUNIX_NET_ABI=%d" % abi, os.path.join(ROOT, "plugins", "net", "unix_net.cc"), "-o", so])
    env = dict(BASE, NCCL_NET_PLUGIN=so, NCCL_DEBUG="INFO", NCCL_DEBUG_SUBSYS="NET,INIT", NCCL_DEBUG_FILE=str(tmp_path / "log.%p"))
    _check(run_ranks(_rank, 3, args=(2,), env=env), 3)
    logs = _logs(tmp_path)
    assert "speaks interface v%d" % abi in logs
    assert "network backend: plugin UnixExample" in logs


TUNER_SRC = r"""
#include <stdio.h>
#include <stdlib.h>
#include "plugin/nccl_tuner.h"
static ncclResult_t tInit(size_t nRanks, size_t nNodes, ncclDebugLogger_t log, void** ctx) { *ctx = malloc(4); return ncclSuccess; }
static ncclResult_t tDestroy(void* ctx) { free(ctx); return ncclSuccess; }
static void note(void) { const char* f = getenv("TUNER_NOTE"); if (f) { FILE* fp = fopen(f, "a"); if (fp) { fputs("asked\n", fp); fclose(fp); } } }
#if TUNER_ABI == 4
static ncclResult_t tInfo(void* ctx, ncclFunc_t c, size_t n, int pipe, float** t, int na, int np, int reg, int* ch) { note(); *ch = 2; return ncclSuccess; }
const ncclTuner_v4_t ncclTunerPlugin_v4 = {"old4", tInit, tInfo, tDestroy};
#elif TUNER_ABI == 3
static ncclResult_t tInfo(void* ctx, ncclFunc_t c, size_t n, int pipe, float** t, int na, int np, int* ch) { note(); *ch = 2; return ncclSuccess; }
const ncclTuner_v3_t ncclTunerPlugin_v3 = {"old3", tInit, tInfo, tDestroy};
#else
static ncclResult_t tInfo(void* ctx, ncclFunc_t c, size_t n, int cn, int nv, int pipe, int* a, int* p, int* ch) {
  note(); *a = NCCL_ALGO_RING; *p = NCCL_PROTO_SIMPLE; *ch = 1; return ncclSuccess;
}
const ncclTuner_v2_t ncclTunerPlugin_v2 = {"old2", tInit, tInfo, tDestroy};
#endif
"""


@pytest.mark.parametrize("abi", [2, 3, 4])
def test_tuner_plugin_of_an_earlier_interface(tmp_path, abi):
    src = tmp_path / "tuner.c"
    src.write_text(TUNER_SRC)
    so = str(tmp_path / ("libtuner_v%d.so" % abi))
    subprocess.check_call(["gcc", "-O1", "-fPIC", "-shared", "-I" + os.path.join(ROOT, "include"), "-I" + CUDA_INC, "-DTUNER_ABI=%d" % abi, str(src), "-o", so])
    env = dict(BASE, NCCL_TUNER_PLUGIN=so, NCCL_DEBUG="INFO", NCCL_DEBUG_SUBSYS="TUNING,INIT", NCCL_DEBUG_FILE=str(tmp_path / "log.%p"),
               TUNER_NOTE=str(tmp_path / "note"))
    _check(run_ranks(_rank, 2, args=(2,), env=env), 2)
    assert "interface v%d" % abi in _logs(tmp_path)


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference tree not present")
def test_reference_example_plugins_load_unchanged(tmp_path):
    """The reference's example net, tuner and profiler plugins, compiled from its tree without edits."""
    net = str(tmp_path / "libnccl-net-example.so")
    tuner = str(tmp_path / "libnccl-tuner-example.so")
    prof = str(tmp_path / "libnccl-profiler-example.so")
    subprocess.check_call(["gcc", "-I" + REF + "/net/example/nccl", "-fPIC", "-shared", "-o", net, REF + "/net/example/plugin.c"])
    subprocess.check_call(["gcc", "-I" + REF + "/tuner/example/nccl", "-fPIC", "-shared", "-o", tuner, REF + "/tuner/example/plugin.c"])
    ex = REF + "/profiler/example"
    subprocess.check_call(["g++", "-std=c++17", "-I" + ex + "/nccl", "-I" + ex, "-I" + CUDA_INC, "-fPIC", "-shared", "-o", prof] +
                          [os.path.join(ex, f) for f in sorted(os.listdir(ex)) if f.endswith(".cc")] + ["-lpthread"])
    env = dict(BASE, NCCL_NET_PLUGIN=net, NCCL_TUNER_PLUGIN=tuner, NCCL_PROFILER_PLUGIN=prof, NCCL_DEBUG="INFO",
               NCCL_DEBUG_SUBSYS="NET,INIT,TUNING,PROFILE", NCCL_DEBUG_FILE=str(tmp_path / "log.%p"), NCCL_PROFILE_DUMP_FILE=str(tmp_path / "trace"))
    _check(run_ranks(_rank, 2, args=(2,), env=env), 2)
    logs = _logs(tmp_path)
    # the example net plugin offers no device: the library says so and stays on its own backend
    assert "found no usable device" in logs or "network backend: plugin" in logs
    assert "tuner plugin" in logs
    assert "profiler plugin" in logs.lower()
