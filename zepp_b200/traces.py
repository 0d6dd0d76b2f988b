"""Routing-trace slices and the deterministic batch sampler of the trace-replay benchmark
(reference: bench/traces.py:1-124; file format: data/traces/manifest.json:1-20).

A trace directory holds `manifest.json` and, per model key, `eval.txt` (the rows batches are drawn
from) and `pool.txt` (the preceding window: the load histogram the placement is planned from).
One text line = the top-k expert ids of one decode token.  A batch draws tokens_per_rank rows per
rank with replacement from one `random.Random` stream in (rank, token) order; the stream's seed is
the 32-bit FNV-1a hash of a key string naming the slice, the topology, the send budget and the row
size, so a batch is a pure function of (slice, ranks, ranks_per_node, budget_mib, chunk_bytes) and
equals the reference's batch for the same trace files.

The reference's own trace files are not shipped with this package: `write_synthetic_slice` writes a
stand-in directory of the same format from a seeded Zipf popularity, and `bench.py --trace-dir`
accepts any directory of this layout.
"""
import hashlib
import json
import os
import random
from dataclasses import dataclass

_FNV_OFFSET = 0x811C9DC5
_FNV_PRIME = 0x01000193


@dataclass(frozen=True)
class TraceSlice:
    model: str            # key in the manifest ("qwen3", "k2")
    trace_model: str      # model name inside the sampler key ("Qwen3-235B", "Kimi-K2")
    num_experts: int
    topk: int
    pool_sha: str         # fingerprint of the full trace set the slice was cut from (part of the seed)
    eval_rows: tuple
    pool_rows: tuple


def read_rows(path):
    """Rows of a trace text file: one tuple of expert ids per non-empty line."""
    rows = []
    with open(path) as fh:
        for line in fh:
            fields = line.split()
            if fields:
                rows.append(tuple(map(int, fields)))
    return tuple(rows)


def load_slice(model, data_dir):
    """Reads `data_dir/manifest.json` and the model's eval / pool files (bench/traces.py:40-49)."""
    with open(os.path.join(data_dir, "manifest.json")) as fh:
        manifest = json.load(fh)
    entry = manifest["models"][model]
    ev = read_rows(os.path.join(data_dir, model, "eval.txt"))
    pool = read_rows(os.path.join(data_dir, model, "pool.txt"))
    if len(ev) != entry["rows"]:
        raise ValueError(f"{model}: eval.txt has {len(ev)} rows, the manifest says {entry['rows']}")
    topk = manifest["topk"]
    for r in ev[:64] + pool[:64]:
        if len(r) != topk or not all(0 <= e < entry["num_experts"] for e in r):
            raise ValueError(f"{model}: malformed trace row {r}")
    return TraceSlice(model, entry["trace_model"], entry["num_experts"], topk, entry["pool_sha"], ev, pool)


def tokens_per_rank(budget_mib, chunk_bytes, topk):
    """Tokens per rank of a pre-top-k send budget of `budget_mib` MiB with `chunk_bytes` token rows: the
    nearest multiple of topk, at least topk (bench/traces.py:52-54; Python's round-half-even)."""
    return max(topk, round(budget_mib * (1 << 20) / (chunk_bytes * topk)) * topk)


def fnv1a32(text):
    h = _FNV_OFFSET
    for byte in text.encode():
        h = ((h ^ byte) * _FNV_PRIME) & 0xFFFFFFFF
    return h


def batch_key(ts, ranks, ranks_per_node, budget_mib, chunk_bytes, instance="001"):
    """The sampler's key string (bench/traces.py:65-75).  Its fixed fields name the trace-generation run
    the slices came from; they must stay as they are for batches to match the reference's."""
    source = "livecodebench/execution"
    fingerprint = hashlib.sha256(f"{source} {ts.pool_sha}".encode()).hexdigest()[:12]
    fields = dict(model=ts.trace_model, layer=5, pool="decode", pools=source, poolsha=fingerprint, sem="homog",
                  dslots="64:32")
    params = ",".join(f"{k}={fields[k]}" for k in sorted(fields))
    budget = int(budget_mib) if float(budget_mib).is_integer() else budget_mib
    return f"trace|{params}|w{ranks}x{ranks_per_node}|b{budget}|k{ts.topk}|c{chunk_bytes}|id{instance}"


def batch_seed(ts, ranks, ranks_per_node, budget_mib, chunk_bytes, instance="001"):
    return fnv1a32(batch_key(ts, ranks, ranks_per_node, budget_mib, chunk_bytes, instance))


def sample_batch(ts, ranks, ranks_per_node, budget_mib, chunk_bytes):
    """ranks * tokens_per_rank rows of top-k ids; row t belongs to rank t // tokens_per_rank
    (bench/traces.py:78-85)."""
    per_rank = tokens_per_rank(budget_mib, chunk_bytes, ts.topk)
    rng = random.Random(batch_seed(ts, ranks, ranks_per_node, budget_mib, chunk_bytes))
    n = len(ts.eval_rows)
    return [ts.eval_rows[rng.randrange(n)] for _ in range(ranks * per_rank)]


def routing_text(rows, topk, num_experts):
    """Canonical text of a batch (header `rows topk experts`, then one row per line): what the
    reference hashes in its self test (bench/traces.py:88-91)."""
    out = [f"{len(rows)} {topk} {num_experts}"]
    out.extend(" ".join(map(str, r)) for r in rows)
    return "\n".join(out) + "\n"


def batch_sha256(ts, ranks, ranks_per_node, budget_mib, chunk_bytes):
    rows = sample_batch(ts, ranks, ranks_per_node, budget_mib, chunk_bytes)
    return hashlib.sha256(routing_text(rows, ts.topk, ts.num_experts).encode()).hexdigest()


def self_test(data_dir, expected):
    """expected: {(model, ranks, ranks_per_node, budget_mib, chunk_bytes): sha256 of the batch text}.
    Returns the list of keys whose regenerated batch hashes differently (bench/traces.py:105-116)."""
    slices = {}
    bad = []
    for key, want in expected.items():
        model = key[0]
        if model not in slices:
            slices[model] = load_slice(model, data_dir)
        if batch_sha256(slices[model], *key[1:]) != want:
            bad.append(key)
    return bad


def pool_routing(ts, ranks, rows_per_rank, topk=None):
    """The pool window as a [ranks, rows_per_rank, topk] nested list (cyclic over the pool rows): the sizing /
    placement input of a layer (the reference plans placement from the pool histogram)."""
    n = len(ts.pool_rows)
    return [[list(ts.pool_rows[(r * rows_per_rank + t) % n]) for t in range(rows_per_rank)] for r in range(ranks)]


def write_synthetic_slice(data_dir, model, trace_model, num_experts, topk, rows, zipf_s, seed):
    """Writes a stand-in slice of the reference's layout: `rows` eval rows and `rows` pool rows of `topk` distinct
    expert ids drawn from a Zipf(zipf_s) popularity over a seeded permutation of the experts."""
    rng = random.Random(seed)
    order = list(range(num_experts))
    rng.shuffle(order)
    weights = [0.0] * num_experts
    for rank_, e in enumerate(order):
        weights[e] = (rank_ + 1.0) ** (-zipf_s)
    os.makedirs(os.path.join(data_dir, model), exist_ok=True)

    def draw():
        picked = []
        w = list(weights)
        for _ in range(topk):
            e = rng.choices(range(num_experts), weights=w)[0]
            picked.append(e)
            w[e] = 0.0
        return picked

    for name in ("pool", "eval"):
        with open(os.path.join(data_dir, model, f"{name}.txt"), "w") as fh:
            for _ in range(rows):
                fh.write(" ".join(map(str, draw())) + "\n")
    pool_sha = hashlib.sha256(f"synthetic {model} {num_experts} {topk} {rows} {zipf_s} {seed}".encode()).hexdigest()
    mpath = os.path.join(data_dir, "manifest.json")
    manifest = {"description": "synthetic stand-in for expert-routing traces", "layer": 5, "topk": topk, "models": {}}
    if os.path.exists(mpath):
        with open(mpath) as fh:
            manifest = json.load(fh)
        if manifest["topk"] != topk:
            raise ValueError("one manifest holds one topk")
    manifest["models"][model] = {"trace_model": trace_model, "num_experts": num_experts, "rows": rows, "pool_sha": pool_sha}
    with open(mpath, "w") as fh:
        json.dump(manifest, fh, indent=1)
    return data_dir
