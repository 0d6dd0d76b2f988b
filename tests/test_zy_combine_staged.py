"""The combine GEMM's line-staged epilogue (ZEPP_B200_COMBINE_STAGED=1: rows staged per warp in shared memory,
whole 128-byte lines stored) under the layer's own parity tests.  The switch is read when a layer is created,
so the parity tests run again in a child process with it set.  Expected to fail rather than failing the suite
until the variant has had its first GPU run: it was written after the GPU budget of its round was spent."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.xfail(strict=False, reason="first GPU run of the line-staged combine epilogue")
def test_layer_parity_with_line_staged_combine_epilogue():
    env = dict(os.environ, ZEPP_B200_COMBINE_STAGED="1")
    sel = "emulated_ranks or odd_number or single_rank_small or many_rows or repeat or trace_replay"
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_layer_gpu.py"), "-m", "gpu",
                        "-x", "-q", "-k", sel], env=env, capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
