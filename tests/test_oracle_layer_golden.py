"""oracle/layer.py against outputs of the reference's own layer check code (tests/golden/make_layer_golden.py):
`examples/serving_check.py:reference` (fp32) and the bf16 loop of `bench/replay.py:torch_reference` around the
reference's `zepp.layer.activation`."""
import os

import numpy as np
import pytest
import torch

from oracle import layer as ol

HERE = os.path.dirname(os.path.abspath(__file__))
Z = np.load(os.path.join(HERE, "golden", "layer_cases.npz"))
N = int(Z["n_cases"][0])


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def _case(i):
    g = lambda k: Z[f"l{i}.{k}"]  # noqa: E731
    return dict(x=_bf16(g("x")), ids=torch.from_numpy(g("ids")), w=torch.from_numpy(g("w")), W1=_bf16(g("W1")),
                W2=_bf16(g("W2")), y_fp32=torch.from_numpy(g("y_fp32")), y_bf16=_bf16(g("y_bf16")), y_gelu=_bf16(g("y_gelu")),
                dims=[int(v) for v in g("dims")])


@pytest.mark.parametrize("i", range(N))
def test_fp32_path_equals_the_reference_check(i):
    c = _case(i)
    y = ol.moe_reference_fp32(c["x"], c["ids"], c["w"], c["W1"], c["W2"])
    assert torch.allclose(y, c["y_fp32"], rtol=1e-5, atol=1e-6), float((y - c["y_fp32"]).abs().max())


@pytest.mark.parametrize("i", range(N))
def test_bf16_rounding_points_equal_the_reference_bf16_loop(i):
    """Same rounding points; the only freedom left is the summation order inside a CPU bf16 matmul, worth at most one
    bf16 step on a few elements."""
    c = _case(i)
    y = ol.moe_reference_bf16_points(c["x"], c["ids"], c["w"], c["W1"], c["W2"]).float()
    ref = c["y_bf16"].float()
    assert torch.allclose(y, ref, rtol=2 ** -7, atol=2e-4), float((y - ref).abs().max())
    assert float((y != ref).float().mean()) < 0.05


@pytest.mark.parametrize("i", range(N))
def test_gelu_path_equals_the_reference_bf16_loop(i):
    c = _case(i)
    ffn = c["dims"][3]
    y = ol.moe_reference_bf16_points(c["x"], c["ids"], c["w"], c["W1"][:, :ffn].contiguous(), c["W2"], act="gelu").float()
    ref = c["y_gelu"].float()
    assert torch.allclose(y, ref, rtol=2 ** -7, atol=2e-4), float((y - ref).abs().max())
