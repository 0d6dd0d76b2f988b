"""The combine GEMM's two epilogue forms under the layer's own parity tests.  The form is chosen when a layer is
created (ZEPP_B200_COMBINE_STAGED: unset = staged lines whenever rows cross to other ranks, "1" = always staged,
"0" = never), so the parity tests run again in child processes with each forced setting."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("forced", ["1", "0"])
def test_layer_parity_with_forced_combine_epilogue(forced):
    env = dict(os.environ, ZEPP_B200_COMBINE_STAGED=forced)
    sel = "emulated_ranks or odd_number or single_rank_small or many_rows or repeat or trace_replay"
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_layer_gpu.py"), "-m", "gpu",
                        "-x", "-q", "-k", sel], env=env, capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
