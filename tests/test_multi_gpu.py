"""The layer across real GPUs (one process per GPU, CUDA IPC, NVLink peer access).  Skipped when
fewer than two GPUs are visible."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _run(nproc, *extra):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "dist_layer_check.py"), *extra]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)


@pytest.mark.parametrize("strategy", ["overlap", "direct"])
def test_layer_across_gpus(strategy):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    nproc = 2 if n < 4 else (4 if n < 8 else 8)
    r = _run(nproc, "--strategy", strategy)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("PASS") == nproc, r.stdout[-3000:]


def test_layer_across_gpus_with_swap():
    """Expert swap across real GPUs: moved experts' weights are pulled over NVLink from the source rank's slots."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    nproc = 2 if n < 4 else (4 if n < 8 else 8)
    r = _run(nproc, "--strategy", "overlap", "--swap", "1", "--steps", "4")
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("PASS") == nproc, r.stdout[-3000:]
