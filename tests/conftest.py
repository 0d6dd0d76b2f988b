import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on a B200)")


class Cases:
    """Prefix-indexed view of one golden .npz (keys `<prefix><i>.<name>`)."""

    def __init__(self, path, prefix, count_key):
        self.z = np.load(path)
        self.prefix = prefix
        self.n = int(self.z[count_key][0])

    def case(self, i):
        pre = f"{self.prefix}{i}."
        return {k[len(pre):]: self.z[k] for k in self.z.files if k.startswith(pre)}


@pytest.fixture(scope="session")
def planner_cases():
    return Cases(os.path.join(GOLDEN, "planner_cases.npz"), "c", "n_cases")


@pytest.fixture(scope="session")
def swap_cases():
    return Cases(os.path.join(GOLDEN, "swap_cases.npz"), "s", "n_seq")


@pytest.fixture(scope="session")
def config_cases():
    return np.load(os.path.join(GOLDEN, "config_cases.npz"))
