"""Seeded synthetic workloads with the shapes and value distributions of the benchmark
configurations (they stand in for the trace-derived batches the reference replays): routing by
expert popularity (uniform or Zipf over a seeded permutation, optional per-step drift), softmax
gate weights, N(0,1) activations, N(0, 0.02) expert weights."""
import dataclasses
import math

import torch

from .config import SHAPES, ModelShape

WORKLOADS = {
    # name: (shape key, tokens/rank, zipf exponent (0 = uniform), router_c, swap)
    "cpu-ref": ("qwen3-30b", 128, 0.0, 0.25, False),
    "qwen3-30b": ("qwen3-30b", 512, 0.0, 0.25, False),
    "qwen3-235b": ("qwen3", 512, 1.0, 0.25, True),
    "k2": ("k2", 512, 1.2, 0.25, True),
}


def shape_of(name) -> ModelShape:
    return dataclasses.replace(SHAPES[WORKLOADS[name][0]], act="swiglu")


def popularity(G, zipf_s, gen):
    """Expert popularity: uniform, or Zipf(s) over a seeded permutation of the experts."""
    if zipf_s == 0:
        return torch.full((G,), 1.0 / G)
    perm = torch.randperm(G, generator=gen)
    p = torch.empty(G)
    p[perm] = (torch.arange(G, dtype=torch.float64) + 1.0).pow(-zipf_s).float()
    return p / p.sum()


def drift(p, frac, gen):
    """Re-permute the popularity among ceil(frac * G) randomly chosen experts."""
    G = p.numel()
    n = math.ceil(frac * G)
    idx = torch.randperm(G, generator=gen)[:n]
    q = p.clone()
    q[idx] = p[idx[torch.randperm(n, generator=gen)]]
    return q


def routing(W, S, K, p, gen):
    """topk_ids [W, S, K] int32 (distinct within a token), topk_weights [W, S, K] fp32 softmax."""
    ids = torch.multinomial(p.expand(W * S, -1), K, replacement=False, generator=gen).int().view(W, S, K)
    wts = torch.softmax(torch.randn(W, S, K, generator=gen), dim=-1)
    return ids, wts


def tokens(rank, S, H, seed=0, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed * 1000 + rank)
    return torch.randn(S, H, generator=g).to(dtype)


def expert_w1(e, shape: ModelShape, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(10007 + e)
    return (0.02 * torch.randn(shape.ffn1, shape.hidden, generator=g)).to(dtype)


def expert_w2(e, shape: ModelShape, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(20011 + e)
    return (0.02 * torch.randn(shape.hidden, shape.ffn_hidden, generator=g)).to(dtype)


def fast_weights(shape: ModelShape, experts, device, seed=7):
    """Device-side N(0, 0.02) weights for many experts at once (benchmark setup; values differ from
    expert_w1/expert_w2 but follow the same distribution).  Returns dict e -> (w1, w2)."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for e in experts:
        w1 = (0.02 * torch.randn(shape.ffn1, shape.hidden, generator=g, device=device)).bfloat16()
        w2 = (0.02 * torch.randn(shape.hidden, shape.ffn_hidden, generator=g, device=device)).bfloat16()
        out[e] = (w1, w2)
    return out


def device_expert(e, shape: ModelShape, device, seed=7):
    """N(0, 0.02) weights (w1 [ffn1, H], w2 [H, I], bf16) of expert e generated on `device`, a function of
    (seed, e) only: any rank can regenerate any expert (benchmark set-up and its sampled parity check)."""
    g = torch.Generator(device=device).manual_seed(seed * 100003 + e)
    w1 = (0.02 * torch.randn(shape.ffn1, shape.hidden, generator=g, device=device)).bfloat16()
    w2 = (0.02 * torch.randn(shape.hidden, shape.ffn_hidden, generator=g, device=device)).bfloat16()
    return w1, w2


def make(name, W, seed=0, S=None):
    """(shape, S, ids [W,S,K], wts [W,S,K], popularity, generator) of a named workload at W ranks."""
    key, S0, zipf_s, _c, _swap = WORKLOADS[name]
    shape = shape_of(name)
    S = S or S0
    gen = torch.Generator().manual_seed(seed)
    p = popularity(shape.num_experts, zipf_s, gen)
    ids, wts = routing(W, S, shape.topk, p, gen)
    return shape, S, ids, wts, p, gen


def from_trace(name, W, data_dir, budget_mib, seed=0):
    """A named workload's shape with routing drawn from a trace directory (zepp_b200/traces.py) instead of
    the synthetic popularity: (shape, S, ids [W,S,K], wts [W,S,K], pool ids [W,S,K], trace model key).
    The batch is the reference sampler's batch for (slice, W ranks on one node, budget, row bytes);
    gate weights are seeded softmax (traces hold expert ids only)."""
    from . import traces
    shape = shape_of(name)
    model = {128: "qwen3", 384: "k2"}[shape.num_experts]
    ts = traces.load_slice(model, data_dir)
    assert ts.topk == shape.topk and ts.num_experts == shape.num_experts, (ts.topk, ts.num_experts)
    chunk = shape.hidden * 2                                   # one bf16 token row
    S = traces.tokens_per_rank(budget_mib, chunk, ts.topk)
    rows = traces.sample_batch(ts, W, W, budget_mib, chunk)
    ids = torch.tensor(rows, dtype=torch.int32).view(W, S, shape.topk)
    gen = torch.Generator().manual_seed(seed)
    wts = torch.softmax(torch.randn(W, S, shape.topk, generator=gen), dim=-1)
    pool = torch.tensor(traces.pool_routing(ts, W, S), dtype=torch.int32)
    return shape, S, ids, wts, pool, model
