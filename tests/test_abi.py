"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""
import os
import re

from zepp_b200._ext import SYMBOLS, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "zepp_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zepp_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = declared_symbols()
    assert len(names) >= 30
    handle = lib()
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in include/zepp_b200.h but not exported"
    assert set(SYMBOLS) == set(names), sorted(set(SYMBOLS) ^ set(names))


def test_size_helpers_need_no_gpu():
    handle = lib()
    assert handle.zepp_abi_version() == 1
    assert handle.zepp_route_workspace_ints(128, 8) > 0
    assert handle.zepp_swap_decide_out_ints(8, 128, 18, 8) == 3 + 8 + 4 * 8 * 8 + 8 * 18 + 128
    # dispatch plan block: header 8, L + NN segments + 1, 3 words per local rank, per-node tables
    assert handle.zepp_dispatch_plan_words(4, 2) == 8 + 6 + 12 + 2 * (6 + 32) + 2 * 7
