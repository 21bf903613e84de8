"""The C / CUDA example programs under examples/: complete users of the public headers and the
shared library (built by make into nccl_b200/bin/examples). Each uses every visible GPU, at most four."""
import os
import subprocess

import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "nccl_b200", "bin", "examples")


@pytest.mark.parametrize("name", ["allreduce_all_devices", "sendrecv_ring", "window_allgather", "device_api_allreduce", "host_allreduce"])
def test_example(name):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    exe = os.path.join(BIN, name)
    assert os.path.exists(exe), "examples are not built: run make"
    env = dict(os.environ, EXAMPLE_GPUS="4", NCCL_DEBUG="WARN", NCCL_B200_WAIT_TIMEOUT_MS="10000", NCCL_B200_DEVCOMM_TIMEOUT_MS="5000")
    p = subprocess.run([exe], env=env, capture_output=True, text=True, timeout=180)
    assert p.returncode == 0, p.stdout + p.stderr
    assert name + ":" in p.stdout and "ok" in p.stdout, p.stdout + p.stderr
