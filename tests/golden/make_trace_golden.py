"""Generates tests/golden/traces/ (a synthetic stand-in trace directory) and tests/golden/trace_cases.json
(what the reference's own sampler, bench/traces.py, returns on that directory).

    python tests/golden/make_trace_golden.py /path/to/reference

The reference's trace files themselves are not copied; as a cross-check the script also runs this
package's sampler on them where they lie and records whether it reproduces the batch hashes the
reference publishes in its self test.
"""
import hashlib
import importlib.util
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from zepp_b200 import traces  # noqa: E402

KEYS = [("qwen3", 16, 4, 1, 8192), ("qwen3", 8, 8, 4, 8192), ("qwen3", 8, 8, 0.5, 4096), ("qwen3", 1, 1, 16, 8192),
        ("k2", 16, 4, 1, 14336), ("k2", 8, 8, 2.5, 14336), ("k2", 2, 2, 4, 14336)]


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <checkout of the reference project>" % sys.argv[0])
    root = sys.argv[1]
    spec = importlib.util.spec_from_file_location("ref_traces", os.path.join(root, "bench", "traces.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)

    out_dir = os.path.join(HERE, "traces")
    if os.path.isdir(out_dir):
        shutil.rmtree(out_dir)
    traces.write_synthetic_slice(out_dir, "qwen3", "Qwen3-235B", 128, 8, 600, 1.0, seed=11)
    traces.write_synthetic_slice(out_dir, "k2", "Kimi-K2", 384, 8, 500, 1.2, seed=12)

    cases = []
    for (model, W, L, b, chunk) in KEYS:
        ts = ref.load_slice(model, out_dir)
        rows = ref.sample_batch(ts, W, L, b, chunk)
        cases.append({"model": model, "ranks": W, "ranks_per_node": L, "budget_mib": b, "chunk_bytes": chunk,
                      "tokens_per_rank": ref.tokens_per_rank(b, chunk, ts.topk),
                      "seed": ref.batch_seed(ts, W, L, b, chunk),
                      "first_rows": [list(r) for r in rows[:3]],
                      "sha256": hashlib.sha256(ref.routing_text(rows, ts.topk, ts.num_experts).encode()).hexdigest()})
    # cross-check on the reference's own slices, read in place
    published = getattr(ref, "_REFERENCE")
    mine_bad = traces.self_test(ref.DATA_DIR, dict(published))
    theirs_bad = ref.self_test()
    record = {"cases": cases,
              "reference_slices_check": {"cells": len(published), "reference_self_test_failures": theirs_bad,
                                         "this_package_failures": len(mine_bad)}}
    with open(os.path.join(HERE, "trace_cases.json"), "w") as fh:
        json.dump(record, fh, indent=1)
    print(json.dumps(record["reference_slices_check"]))


if __name__ == "__main__":
    main()
