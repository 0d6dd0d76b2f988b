"""Host-side logic of the package on CPU: placement against the reference's golden vectors, the
config / capacity API, the synthetic workload generators."""
import dataclasses

import numpy as np
import pytest
import torch

from zepp_b200 import SHAPES, EPMoEConfig, ModelShape, tokens_per_rank
from zepp_b200 import workloads as wl
from zepp_b200.capacity import CapacityExceeded, Demands, grow, violations
from zepp_b200.placement import demand_histogram, rebuild_l2p, solve_placement
from zepp_b200.routing import Capacities, c_rational, virtual_route
from zepp_b200.swap import parse_swap_block


def test_placement_matches_reference_golden(planner_cases):
    for i in range(planner_cases.n):
        c = planner_cases.case(i)
        R, L, G, K, S, nlp, _, _ = [int(v) for v in c["dims"]]
        pl = solve_placement(demand_histogram(torch.from_numpy(c["pool"]), L, G), L, nlp)
        assert np.array_equal(pl.p2l.numpy(), c["p2l"]), i
        assert np.array_equal(pl.l2p.numpy(), c["l2p"]), i
        assert np.array_equal(pl.lcnts.numpy(), c["lcnts"]), i
        assert np.array_equal(rebuild_l2p(pl.p2l, G, R).numpy(), c["l2p"]), i


def test_config_surface():
    assert SHAPES["qwen3"] == ModelShape(128, 8, 4096, 1536) and SHAPES["k2"] == ModelShape(384, 8, 7168, 2048)
    assert SHAPES["qwen3"].act == "gelu" and SHAPES["qwen3"].ffn1 == 1536
    sw = dataclasses.replace(SHAPES["qwen3"], act="swiglu")
    assert sw.ffn1 == 3072 and sw.chunk_bytes == 8192
    # python/zepp/config.py:27-31: 4 MiB -> 512 tokens (qwen3), 296 (k2)
    assert tokens_per_rank(4, SHAPES["qwen3"]) == 512 and tokens_per_rank(4, SHAPES["k2"]) == 296
    assert tokens_per_rank(1, SHAPES["qwen3"]) == 128 and tokens_per_rank(16, SHAPES["k2"]) == 1168
    cfg = EPMoEConfig(shape=sw, ranks=8, ranks_per_node=8, max_tokens_per_rank=512)
    assert (cfg.slots_per_rank, cfg.groups_per_rank, cfg.virtual_experts, cfg.nodes) == (18, 19, 152, 1)
    with pytest.raises(AssertionError):
        EPMoEConfig(shape=sw, ranks=3, ranks_per_node=3, max_tokens_per_rank=512)
    with pytest.raises(AssertionError):
        EPMoEConfig(shape=sw, ranks=8, ranks_per_node=8, max_tokens_per_rank=12)
    with pytest.raises(AssertionError):
        EPMoEConfig(shape=sw, ranks=8, ranks_per_node=8, max_tokens_per_rank=512, comm_strategy="ring")


def test_slack_rational():
    assert c_rational(0.25) == (1, 4) and c_rational(0.0) == (0, 1) and c_rational(0.5) == (1, 2)
    with pytest.raises(AssertionError):
        c_rational(0.1)


def test_capacity_api():
    caps = Capacities(100, 100, 10, 10, 100, 10, 10, 50)
    d = Demands(120, 90, 1, 1, 1, 1, 60)
    v = violations(d, caps)
    assert [f for f, _, _ in v] == ["recv_cap", "combine_send"]
    assert [f for f, _, _ in violations(d, caps, direct=True)] == ["recv_cap", "pair_cap"]
    g = grow(caps, d)
    assert g.recv_cap == 180 and g.combine_send == 180 and g.dispatch_recv == 180 and g.pair_cap == 50
    assert grow(caps, d, direct=True).pair_cap == 90
    e = CapacityExceeded(v, d)
    assert "recv_cap needs 120 > 100" in str(e)


def test_virtual_route_and_block_parse():
    phys = torch.tensor([[0, 17, 18, 35]])
    assert virtual_route(phys, 18, 19).tolist() == [[1, 18, 20, 37]]
    R, nlp, G, cap = 2, 3, 4, 8
    blk = np.zeros(3 + R + 4 * R * cap + R * nlp + G, dtype=np.int64)
    blk[0], blk[1], blk[3] = 1, 1, 1
    blk[3 + R:3 + R + 4] = [2, 1, 0, 3]
    out = parse_swap_block(blk, R, nlp, G, cap)
    assert out["rounds"] == 1 and out["moves"] == [[(2, 1, 0, 3)], []]


def test_workload_generators_are_seeded(config_cases):
    shape, S, ids, wts, p, _ = wl.make("qwen3-235b", 8)
    assert (shape.hidden, shape.ffn_hidden, shape.act, S) == (4096, 1536, "swiglu", 512)
    assert np.array_equal(ids.numpy(), config_cases["qwen235b_w8.topk"].astype(np.int32))
    assert torch.allclose(wts.sum(-1), torch.ones(8, 512))
    assert all(len(set(row)) == 8 for row in ids.view(-1, 8)[:64].tolist())
    _, _, ids2, _, _, _ = wl.make("qwen3-235b", 8)
    assert torch.equal(ids, ids2)
    g = torch.Generator().manual_seed(3)
    q = wl.drift(p, 0.1, g)
    assert torch.allclose(q.sort().values, p.sort().values) and int((q != p).sum()) <= 13
    assert wl.expert_w1(3, shape).shape == (3072, 4096) and wl.expert_w2(3, shape).shape == (4096, 1536)


def test_token_buckets_follow_the_serving_rule():
    """k, 2k, 4k, ... and max_tokens_per_rank itself (python/zepp/serving.py:42-50), also when the maximum is no power of two."""
    from zepp_b200 import token_buckets
    shape = ModelShape(16, 4, 256, 128, act="swiglu")
    mk = lambda s: EPMoEConfig(shape=shape, ranks=2, ranks_per_node=2, max_tokens_per_rank=s)  # noqa: E731
    assert token_buckets(mk(4)) == [4]
    assert token_buckets(mk(64)) == [4, 8, 16, 32, 64]
    assert token_buckets(mk(40)) == [4, 8, 16, 32, 40]


def test_grow_never_shrinks_and_keeps_the_aliased_buffers_together():
    caps = Capacities(100, 100, 10, 10, 100, 10, 10, 50)
    d = Demands(recv_rows=200, dispatch_recv=90, dispatch_stage=5, dispatch_relay=1, combine_conv=1, combine_wire=1, pair_rows=80)
    g = grow(caps, d)
    assert g.recv_cap == 300 and g.combine_send == 300 and g.dispatch_recv == 300
    assert g.dispatch_stage == 10 and g.pair_cap == 50            # untouched where the demand fits / is not checked
    assert grow(caps, d, direct=True).pair_cap == 120
