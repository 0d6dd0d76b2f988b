"""Trace slices and the deterministic batch sampler against what the reference's own sampler
(bench/traces.py) returned on the committed synthetic slices (tests/golden/make_trace_golden.py)."""
import json
import os

import pytest

from zepp_b200 import traces

HERE = os.path.dirname(os.path.abspath(__file__))
DATA = os.path.join(HERE, "golden", "traces")
with open(os.path.join(HERE, "golden", "trace_cases.json")) as _fh:
    GOLDEN = json.load(_fh)


def test_fnv1a_known_answers():
    assert traces.fnv1a32("") == 0x811C9DC5
    assert traces.fnv1a32("a") == 0xE40C292C
    assert traces.fnv1a32("foobar") == 0xBF9CF968


@pytest.mark.parametrize("case", GOLDEN["cases"], ids=lambda c: f"{c['model']}-w{c['ranks']}x{c['ranks_per_node']}-b{c['budget_mib']}")
def test_batches_equal_the_reference_samplers(case):
    ts = traces.load_slice(case["model"], DATA)
    key = (case["ranks"], case["ranks_per_node"], case["budget_mib"], case["chunk_bytes"])
    assert traces.tokens_per_rank(case["budget_mib"], case["chunk_bytes"], ts.topk) == case["tokens_per_rank"]
    assert traces.batch_seed(ts, *key) == case["seed"]
    rows = traces.sample_batch(ts, *key)
    assert len(rows) == case["ranks"] * case["tokens_per_rank"]
    assert [list(r) for r in rows[:3]] == case["first_rows"]
    assert traces.batch_sha256(ts, *key) == case["sha256"]


def test_the_generating_run_reproduced_the_reference_published_hashes():
    chk = GOLDEN["reference_slices_check"]
    assert chk["cells"] == 6 and chk["reference_self_test_failures"] == 0 and chk["this_package_failures"] == 0


def test_self_test_reports_a_changed_batch():
    c = GOLDEN["cases"][0]
    key = (c["model"], c["ranks"], c["ranks_per_node"], c["budget_mib"], c["chunk_bytes"])
    assert traces.self_test(DATA, {key: c["sha256"]}) == []
    assert traces.self_test(DATA, {key: "0" * 64}) == [key]


def test_tokens_per_rank_rounding():
    assert traces.tokens_per_rank(1, 8192, 8) == 128
    assert traces.tokens_per_rank(1, 14336, 8) == 72          # 73.14 -> 9 x 8
    assert traces.tokens_per_rank(0.001, 8192, 8) == 8        # never below topk
    assert traces.tokens_per_rank(16, 14336, 8) == 1168


def test_synthetic_writer_is_deterministic_and_loadable(tmp_path):
    a = traces.write_synthetic_slice(str(tmp_path / "a"), "qwen3", "Qwen3-235B", 128, 8, 50, 1.0, seed=11)
    b = traces.write_synthetic_slice(str(tmp_path / "b"), "qwen3", "Qwen3-235B", 128, 8, 50, 1.0, seed=11)
    ta, tb = traces.load_slice("qwen3", a), traces.load_slice("qwen3", b)
    assert ta.eval_rows == tb.eval_rows and ta.pool_rows == tb.pool_rows and len(ta.eval_rows) == 50
    assert all(len(set(r)) == 8 for r in ta.eval_rows)
    # the committed slice came from the same call
    gold = traces.load_slice("qwen3", DATA)
    assert gold.eval_rows[:50] == ta.eval_rows[:50] or len(gold.eval_rows) == 600


def test_malformed_slices_are_refused(tmp_path):
    d = traces.write_synthetic_slice(str(tmp_path / "t"), "k2", "Kimi-K2", 384, 8, 20, 1.2, seed=3)
    with open(os.path.join(d, "k2", "eval.txt"), "a") as fh:
        fh.write("1 2 3 4 5 6 7 8\n")
    with pytest.raises(ValueError):
        traces.load_slice("k2", d)          # row count differs from the manifest


def test_pool_routing_shape():
    ts = traces.load_slice("k2", DATA)
    pool = traces.pool_routing(ts, 4, 16)
    assert len(pool) == 4 and len(pool[0]) == 16 and len(pool[0][0]) == 8
