"""The router's vacate pass (one warp, tokens in order) keeps its release / extra budget tables in shared memory when
they fit; a large expert count leaves them in global memory, read through volatile loads and changed by global
atomics.  ZEPP_B200_VACATE_STAGED=0 forces that second form, so the golden routing cases (bit-exact `phys`, budgets
invariant under the pass) and the capacity sizing on the benchmark routings run again in a child process with it."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_vacate_with_tables_in_global_memory():
    env = dict(os.environ, ZEPP_B200_VACATE_STAGED="0")
    cmd = [sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_planner_gpu.py"), "-m", "gpu", "-x", "-q",
           "-k", "route_against_golden or capacities_against_golden"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1200, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
