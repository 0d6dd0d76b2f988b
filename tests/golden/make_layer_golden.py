"""Generates tests/golden/layer_cases.npz: outputs of the reference's own layer check code on small
seeded inputs, to pin oracle/layer.py.

    python tests/golden/make_layer_golden.py /path/to/reference

* `y_fp32`  = examples/serving_check.py `reference(x, ids, w, W1, W2, shape)` run as it is (CPU tensors).
* `y_bf16`  = the loop of bench/replay.py `torch_reference` (which is written for CUDA tensors) re-run here on
  CPU tensors around the reference's own `zepp.layer.activation`: per expert
  `activation(x[rows] @ w1.t(), shape) @ w2.t()` in bf16, fp32 `index_add_` of `part * prob`, one final cast.
* `y_gelu`  = the same loop with a GELU shape.
The reference's `zepp` package loads a compiled extension at import; `zepp._ext` is stubbed as in make_golden.py.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load(root):
    ext = types.ModuleType("zepp._ext")
    ext.C = None
    ext.ensure_shm = lambda group: None
    sys.modules["zepp._ext"] = ext
    sys.path.insert(0, os.path.join(root, "python"))
    import zepp
    from zepp.layer import activation
    spec = importlib.util.spec_from_file_location("ref_serving_check", os.path.join(root, "examples", "serving_check.py"))
    chk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(chk)
    return zepp, activation, chk


@torch.no_grad()
def bf16_loop(activation, x, ids, probs, W1, W2, shape):
    S, K = ids.shape
    y = torch.zeros(S, shape.hidden, dtype=torch.float32)
    e_flat = ids.reshape(-1).long()
    t_flat = torch.arange(S).repeat_interleave(K)
    p_flat = probs.reshape(-1).float()
    for e in torch.unique(e_flat).tolist():
        sel = (e_flat == e).nonzero(as_tuple=True)[0]
        rows = t_flat[sel]
        part = activation(x[rows] @ W1[e].t(), shape) @ W2[e].t()
        y.index_add_(0, rows, part.float() * p_flat[sel].unsqueeze(1))
    return y.to(x.dtype)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <checkout of the reference project>" % sys.argv[0])
    root = sys.argv[1]
    zepp, activation, chk = load(root)
    out = {}
    cases = [(16, 4, 64, 32, 24, 1), (32, 8, 64, 32, 40, 2), (8, 2, 128, 64, 17, 3)]
    for i, (G, K, H, I, n, seed) in enumerate(cases):
        g = torch.Generator().manual_seed(seed)
        shape = zepp.ModelShape(G, K, H, I, act="swiglu")
        gelu = zepp.ModelShape(G, K, H, I, act="gelu")
        x = torch.randn(n, H, generator=g).to(torch.bfloat16)
        ids = torch.multinomial(torch.ones(n, G), K, replacement=False, generator=g).int()
        w = torch.softmax(torch.randn(n, K, generator=g), dim=-1)
        W1 = (0.05 * torch.randn(G, 2 * I, H, generator=g)).to(torch.bfloat16)
        W2 = (0.05 * torch.randn(G, H, I, generator=g)).to(torch.bfloat16)
        y32 = chk.reference(x, ids, w, W1, W2, shape)
        y16 = bf16_loop(activation, x, ids, w, W1, W2, shape)
        yg = bf16_loop(activation, x, ids, w, W1[:, :I].contiguous(), W2, gelu)
        for k, v in (("x", x), ("ids", ids), ("w", w), ("W1", W1), ("W2", W2), ("y_fp32", y32), ("y_bf16", y16),
                     ("y_gelu", yg)):
            # bf16 tensors are stored as their 16-bit patterns
            out[f"l{i}.{k}"] = v.view(torch.int16).numpy() if v.dtype == torch.bfloat16 else v.numpy()
        out[f"l{i}.dims"] = np.array([G, K, H, I, n], dtype=np.int64)
    out["n_cases"] = np.array([len(cases)], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "layer_cases.npz"), **out)
    print("layer cases:", len(cases))


if __name__ == "__main__":
    main()
