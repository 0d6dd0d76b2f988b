"""CPU oracle of the MoE layer arithmetic (TEST INFRASTRUCTURE, not product code).

`moe_reference_fp32` restates the reference's fp32 SwiGLU check path
(examples/serving_check.py:86-99): for every expert, gather the rows that picked it, one
gate|up projection, silu(gate) * up, the down projection, times the top-k weight, summed into
the token's output row.  It is also the CPU baseline that bench.py times.

`moe_reference_bf16_points` follows the rounding points of the reference's bf16 check path
(bench/replay.py:68-83 with python/zepp/layer.py:20-27): bf16 GEMM outputs, bf16 silu, bf16
product, bf16 down projection, fp32 weighted sum, one final rounding.

The reference holds no golden vectors for layer outputs (its checks are tolerance checks against
these torch paths).  Both functions are pinned to outputs of the reference's own check code on small
seeded inputs: tests/golden/layer_cases.npz, made by tests/golden/make_layer_golden.py, which runs
examples/serving_check.py `reference` as it is and the bf16 loop of bench/replay.py around the
reference's `zepp.layer.activation` (tests/test_oracle_layer_golden.py).  The planner oracle beside it
is pinned bit for bit by golden vectors.
"""
import torch


def swiglu_fp32(h, ffn):
    return torch.nn.functional.silu(h[:, :ffn]) * h[:, ffn:]


@torch.no_grad()
def moe_reference_fp32(x, ids, w, W1, W2):
    """x [n, H]; ids [n, K] expert ids (negative: a pad copy, skipped); w [n, K] fp32; W1 [E, 2I, H]; W2 [E, H, I]
    (tensors, or dicts holding the experts that occur) -> y fp32 [n, H]."""
    n, K = ids.shape
    H = x.shape[1]
    xf = x.float()
    y = torch.zeros(n, H, dtype=torch.float32)
    ids = ids.long()
    for e in sorted(set(ids.reshape(-1).tolist())):
        if e < 0:
            continue
        rows, ks = (ids == e).nonzero(as_tuple=True)
        ffn = W1[e].shape[0] // 2
        h = xf[rows] @ W1[e].float().t()
        a = swiglu_fp32(h, ffn)
        y.index_add_(0, rows, (a @ W2[e].float().t()) * w[rows, ks].float().unsqueeze(1))
    return y


@torch.no_grad()
def moe_reference_bf16_points(x, ids, w, W1, W2, act="swiglu"):
    """Same layer with the bf16 rounding points of the reference's bf16 check path; inputs bf16
    tensors (W1/W2 may be given as dicts or tensors indexed by expert).  act="gelu": W1 is [*, I, H] and the
    activation is the exact (erf) GELU on the bf16 projection (python/zepp/layer.py:22-23)."""
    n, K = ids.shape
    H = x.shape[1]
    y = torch.zeros(n, H, dtype=torch.float32)
    ids = ids.long()
    bf = torch.bfloat16
    for e in torch.unique(ids).tolist():
        if e < 0:
            continue
        rows, ks = (ids == e).nonzero(as_tuple=True)
        w1, w2 = W1[e].float(), W2[e].float()
        h = (x[rows].float() @ w1.t()).to(bf)
        if act == "gelu":
            a = torch.nn.functional.gelu(h.float()).to(bf)
        else:
            ffn = w1.shape[0] // 2
            g = torch.nn.functional.silu(h[:, :ffn].float()).to(bf)
            a = (g.float() * h[:, ffn:].float()).to(bf)
        part = (a.float() @ w2.t()).to(bf)
        y.index_add_(0, rows, part.float() * w[rows, ks].float().unsqueeze(1))
    return y.to(bf)
