"""The CTA-pair form of the two grouped GEMMs (256-row token tiles, tcgen05.mma.cta_group::2) under the layer's own
parity tests.  A layer picks the pair kernels by its row count per expert; ZEPP_B200_PAIRS=1 / 0 forces them on /
off when the layer is created, so the parity tests run again in child processes with each forced setting (small
shapes, ragged and multi-tile experts, emulated ranks with the fused gather, the benchmark shapes)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(forced, files, sel):
    env = dict(os.environ, ZEPP_B200_PAIRS=forced)
    cmd = [sys.executable, "-m", "pytest", *[os.path.join(ROOT, "tests", f) for f in files], "-m", "gpu", "-x", "-q", "-k", sel]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1200, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


def test_layer_parity_on_cta_pairs():
    _run("1", ["test_layer_gpu.py"],
         "single_rank_small or many_rows or odd_number or emulated_ranks or repeat or swap_moves or full_size or capacity_violation")


def test_benchmark_shapes_and_buckets_on_cta_pairs():
    _run("1", ["test_layer_shapes_gpu.py"], "eight_emulated_ranks or buckets or pad_rows or wait_that_runs_out")


def test_layer_parity_without_cta_pairs():
    _run("0", ["test_layer_gpu.py"], "many_rows or emulated_ranks_one_node or full_size")
