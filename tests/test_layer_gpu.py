"""The MoE layer through the public API (EPMoE over the C-ABI) against the CPU oracle: planner products
bit-exact; outputs within the stated rtol 2e-2 / atol 2e-2 of the fp32 reference path AND, because the outputs
of N(0, 0.02) weights are themselves of the order of the tolerance, within a scale-aware bound of the oracle's
bf16 path (same rounding points as the kernels): max |err| <= 1.5 % of the largest reference magnitude and a
relative Frobenius error <= 0.5 %.  A halved output, a dropped expert contribution or a zeroed expert fail the
second bound."""
import dataclasses

import numpy as np
import pytest
import torch

from oracle import layer as ol
from oracle import planner as op
from zepp_b200 import EPMoE, EPMoEConfig, ModelShape
from zepp_b200 import workloads as wl
from zepp_b200.capacity import CapacityExceeded
from zepp_b200.layer import LocalGroup, local_step, make_local_layers, token_buckets
from zepp_b200.routing import Capacities

pytestmark = pytest.mark.gpu
RTOL = ATOL = 2e-2            # the reference's check-path tolerance (bench/replay.py:154, examples/serving_check.py:353)
MAX_REL_TO_SCALE = 1.5e-2     # against the bf16-points oracle, relative to max |reference|
FRO_REL = 5e-3


def _weights(shape):
    W1 = torch.stack([wl.expert_w1(e, shape) for e in range(shape.num_experts)])
    W2 = torch.stack([wl.expert_w2(e, shape) for e in range(shape.num_experts)])
    return W1, W2


def _close(y, x, ids, wts, W1, W2, tag, act="swiglu"):
    """y (device or host, any float dtype) against both oracle paths on the same inputs."""
    y = y.float().cpu()
    if act == "swiglu":
        ref32 = ol.moe_reference_fp32(x, ids, wts, W1, W2)
        bad = ~torch.isclose(y, ref32, rtol=RTOL, atol=ATOL)
        assert not bool(bad.any()), f"{tag}: {int(bad.sum())} of {bad.numel()} elements out of rtol/atol 2e-2, " \
                                   f"max |err| {float((y - ref32).abs().max()):.4g}"
    refb = ol.moe_reference_bf16_points(x, ids, wts, W1, W2, act=act).float()
    scale = float(refb.abs().max())
    err = float((y - refb).abs().max())
    fro = float((y - refb).norm() / refb.norm().clamp_min(1e-30))
    assert scale > 0 and err <= MAX_REL_TO_SCALE * scale and fro <= FRO_REL, \
        f"{tag}: max |err| {err:.4g} vs scale {scale:.4g} (limit {MAX_REL_TO_SCALE * scale:.4g}), relative Frobenius {fro:.4g}"


def _check_all(ys, xs, ids, wts, W1, W2, tag):
    for r in range(len(xs)):
        _close(ys[r], xs[r], ids[r], wts[r], W1, W2, f"{tag} rank{r}")


def _run_local(shape, W, L, S, strategy, zipf=0.0, seed=0, steps=2, check_plan=True):
    cfg = EPMoEConfig(shape=shape, ranks=W, ranks_per_node=L, max_tokens_per_rank=S, comm_strategy=strategy)
    gen = torch.Generator().manual_seed(seed)
    p = wl.popularity(shape.num_experts, zipf, gen)
    ids, wts = wl.routing(W, S, shape.topk, p, gen)
    layers, rts = make_local_layers(cfg, ids, ids, wait_limit_ms=500)
    W1, W2 = _weights(shape)
    for l in layers:
        l.load_weights(lambda e: W1[e], lambda e: W2[e])
    try:
        for step in range(steps):
            if step:
                ids, wts = wl.routing(W, S, shape.topk, p, gen)
            xs = [wl.tokens(r, S, shape.hidden, seed=seed + 10 * step) for r in range(W)]
            ys = local_step(layers, [ids[r].cuda() for r in range(W)], [wts[r].cuda() for r in range(W)],
                            [x.cuda() for x in xs])
            for l in layers:
                l.check()
            _check_all(ys, xs, ids, wts, W1, W2, f"{strategy} W{W} L{L} step{step}")
            if check_plan:
                pl0 = layers[0].placement
                pl = op.Placement(pl0.p2l.numpy(), pl0.l2p.numpy(), pl0.lcnts.numpy())
                phys, _ = op.reference_route(ids.numpy(), pl, cfg.slots_per_rank, L, cfg.router_c)
                vce = op.virtual_route(phys.reshape(W * S, -1), cfg.slots_per_rank, cfg.groups_per_rank)
                splits, scat, sps, uc = op.routed_meta(vce, W, S, cfg.groups_per_rank, W // L, L)
                for r, l in enumerate(layers):
                    t = dict(zip(("vce", "splits", "scatter_index", "sps", "uc", "phys_own", "m_this"),
                                 l.tables("vce", "splits", "scatter_index", "sps", "uc", "phys_own", "m_this")))
                    assert np.array_equal(t["phys_own"].cpu().numpy().reshape(S, -1), phys[r]), (r, "phys")
                    assert np.array_equal(t["vce"].cpu().numpy().reshape(vce.shape), vce), (r, "vce")
                    assert np.array_equal(t["splits"].cpu().numpy(), splits), (r, "splits")
                    assert np.array_equal(t["scatter_index"].cpu().numpy().reshape(scat.shape), scat), (r, "scatter")
                    assert np.array_equal(t["sps"].cpu().numpy().reshape(sps.shape), sps), (r, "sps")
                    assert np.array_equal(t["uc"].cpu().numpy().reshape(uc.shape), uc), (r, "uc")
                    gpe = cfg.groups_per_rank
                    assert int(t["m_this"][0]) == int(splits[r * gpe:(r + 1) * gpe].sum())
                    words, head = op.dispatch_plan_head(sps, uc, W, L, gpe, r, S * cfg.shape.topk, layers[r].caps.dispatch_recv)
                    assert l.tables("dplan")[0].cpu().tolist()[:head] == words[:head], (r, "dplan")
                    if W == L:
                        so, sr, do, lo = op.combine_tables(sps, W, gpe, r)
                        assert l.tables("cplan")[0].cpu().tolist() == np.concatenate([so, sr, do, lo]).tolist(), (r, "cplan")
    finally:
        for l in layers:
            l.close()
        for rt in rts:
            rt.destroy()


SMALL = ModelShape(16, 4, 256, 128, act="swiglu")
MID = ModelShape(32, 8, 512, 256, act="swiglu")


@pytest.mark.parametrize("strategy", ["direct", "overlap"])
def test_single_rank_small(strategy):
    _run_local(SMALL, 1, 1, 32, strategy)


@pytest.mark.parametrize("strategy", ["direct", "overlap"])
def test_single_rank_many_rows_per_expert(strategy):
    """More than one 128-row token tile per expert and ragged last tiles."""
    _run_local(SMALL, 1, 1, 1000, strategy, zipf=1.0, steps=1)


@pytest.mark.parametrize("strategy", ["direct", "overlap"])
def test_hidden_with_an_odd_number_of_feature_blocks(strategy):
    """hidden = 3 x 128: the combine GEMM's last item of an expert has only one of its two feature blocks."""
    _run_local(ModelShape(16, 4, 384, 128, act="swiglu"), 2, 2, 200, strategy, zipf=1.0, steps=1)


@pytest.mark.parametrize("strategy", ["direct", "overlap"])
def test_single_rank_gelu(strategy):
    shape = ModelShape(16, 4, 256, 128, act="gelu")
    cfg = EPMoEConfig(shape=shape, ranks=1, ranks_per_node=1, max_tokens_per_rank=64, comm_strategy=strategy)
    gen = torch.Generator().manual_seed(3)
    ids, wts = wl.routing(1, 64, 4, wl.popularity(16, 0.0, gen), gen)
    layer = EPMoE(cfg, LocalGroup(0, 1), ids, ids)
    W1, W2 = _weights(shape)
    layer.load_weights(lambda e: W1[e], lambda e: W2[e])
    x = wl.tokens(0, 64, 256)
    plan = layer.prepare(ids[0].cuda(), wts[0].cuda())
    y = layer.forward(x.cuda(), plan)
    layer.check()
    ref = torch.zeros(64, 256)
    for t in range(64):
        for j in range(4):
            e = int(ids[0, t, j])
            h = torch.nn.functional.gelu(x[t].float() @ W1[e].float().t())
            ref[t] += float(wts[0, t, j]) * (h @ W2[e].float().t())
    assert torch.allclose(y.float().cpu(), ref, rtol=RTOL, atol=ATOL)
    _close(y, x, ids[0], wts[0], W1, W2, f"gelu {strategy}", act="gelu")
    layer.close()


@pytest.mark.parametrize("strategy", ["direct", "overlap"])
@pytest.mark.parametrize("W,L", [(2, 2), (4, 4), (8, 8)])
def test_emulated_ranks_one_node(strategy, W, L):
    _run_local(MID, W, L, 64, strategy, zipf=1.0 if W == 4 else 0.0)


@pytest.mark.parametrize("W,L", [(4, 2), (8, 4), (8, 2)])
def test_emulated_ranks_virtual_nodes(W, L):
    """Replicated experts, capacity routing and the vacate pass (virtual nodes on one box)."""
    _run_local(MID, W, L, 64, "overlap", zipf=1.0, seed=2)


def test_fresh_payload_each_step_and_bitwise_repeat():
    """A new x every step (a stale-delivery bug cannot pass, bench/replay.py:141-143) and identical
    outputs when a step is repeated (deterministic combine)."""
    shape, W, S = MID, 2, 64
    cfg = EPMoEConfig(shape=shape, ranks=W, ranks_per_node=W, max_tokens_per_rank=S)
    gen = torch.Generator().manual_seed(11)
    ids, wts = wl.routing(W, S, shape.topk, wl.popularity(shape.num_experts, 0.0, gen), gen)
    layers, rts = make_local_layers(cfg, ids, ids, wait_limit_ms=500)
    W1, W2 = _weights(shape)
    for l in layers:
        l.load_weights(lambda e: W1[e], lambda e: W2[e])
    idc, wtc = [ids[r].cuda() for r in range(W)], [wts[r].cuda() for r in range(W)]
    outs = []
    for step in (0, 1, 0):
        xs = [wl.tokens(r, S, shape.hidden, seed=step) for r in range(W)]
        ys = local_step(layers, idc, wtc, [x.cuda() for x in xs])
        _check_all(ys, xs, ids, wts, W1, W2, f"step {step}")
        outs.append([y.clone() for y in ys])
    for r in range(W):
        assert torch.equal(outs[0][r], outs[2][r])
        assert not torch.equal(outs[0][r], outs[1][r])
    for l in layers:
        l.check()
        l.close()
    for rt in rts:
        rt.destroy()


def test_capacity_violation_is_reported_not_faulted():
    """A receive capacity one row short of the demand: the device mask names the buffers, the GEMMs
    compute nothing, the host raises CapacityExceeded and the context stays usable."""
    shape, S = SMALL, 32
    cfg = EPMoEConfig(shape=shape, ranks=1, ranks_per_node=1, max_tokens_per_rank=S)
    gen = torch.Generator().manual_seed(0)
    ids, wts = wl.routing(1, S, shape.topk, wl.popularity(shape.num_experts, 0.0, gen), gen)
    tight = Capacities(*([S * shape.topk - 1] * 8))
    import zepp_b200.layer as zl
    orig = zl.compute_capacities
    zl.compute_capacities = lambda *a, **k: tight
    try:
        layer = EPMoE(cfg, LocalGroup(0, 1), ids, ids)
    finally:
        zl.compute_capacities = orig
    W1, W2 = _weights(shape)
    layer.load_weights(lambda e: W1[e], lambda e: W2[e])
    plan = layer.prepare(ids[0].cuda(), wts[0].cuda())
    y = layer.forward(wl.tokens(0, S, shape.hidden).cuda(), plan)
    with pytest.raises(CapacityExceeded) as ei:
        layer.check()
    assert {f for f, _, _ in ei.value.violations} >= {"recv_cap", "combine_send"}
    assert float(y.float().abs().max()) == 0.0
    assert float(torch.ones(3, device="cuda").sum()) == 3.0
    layer.close()


def test_benchmark_shape_one_rank_of_eight():
    """Qwen3-30B layer shape, 8-way sharding emulated on one GPU at 64 tokens per rank (full H, I, E)."""
    shape = dataclasses.replace(wl.shape_of("qwen3-30b"))
    _run_local(shape, 8, 8, 64, "overlap", steps=1, check_plan=False)


def test_swap_moves_weights_and_routes_on_the_new_placement():
    """swap=True on 8 emulated ranks with skewed routing: the device decision equals the host oracle's, the
    placement tables change, the moved experts' weights follow them, and outputs stay within tolerance on the
    swap step and on the steps after it."""
    shape, W, S = MID, 8, 64
    cfg = EPMoEConfig(shape=shape, ranks=W, ranks_per_node=W, max_tokens_per_rank=S, swap=True)
    gen = torch.Generator().manual_seed(4)
    p = wl.popularity(shape.num_experts, 1.2, gen)
    ids, wts = wl.routing(W, S, shape.topk, p, gen)
    layers, rts = make_local_layers(cfg, ids, ids, wait_limit_ms=500)
    W1, W2 = _weights(shape)
    for l in layers:
        l.load_weights(lambda e: W1[e], lambda e: W2[e])
    pl0 = layers[0].placement
    cur = op.Placement(pl0.p2l.numpy().copy(), pl0.l2p.numpy().copy(), pl0.lcnts.numpy())
    total_moves = 0
    try:
        for step in range(3):
            if step == 2:
                p = wl.drift(p, 0.5, gen)
            if step:
                ids, wts = wl.routing(W, S, shape.topk, p, gen)
            xs = [wl.tokens(r, S, shape.hidden, seed=step) for r in range(W)]
            ys = local_step(layers, [ids[r].cuda() for r in range(W)], [wts[r].cuda() for r in range(W)],
                            [x.cuda() for x in xs])
            for l in layers:
                l.check()
            load_g = np.bincount(ids.numpy().reshape(-1), minlength=shape.num_experts)
            new, rounds = op.decide_swaps(load_g, cur, W, cfg.slots_per_rank, cfg.router_c)
            if rounds:
                moves = op.net_moves(cur.p2l, new, W, cfg.slots_per_rank)
                total_moves += sum(len(m) for m in moves)
                cur = op.Placement(new, op.rebuild_l2p(new, shape.num_experts, W), cur.lcnts)
                assert layers[0].swap_moves == sum(len(m) for m in moves)
            else:
                assert layers[0].swap_moves == 0
            for l in layers:
                assert np.array_equal(l.tables("p2l")[0].cpu().numpy(), cur.p2l), step
            _check_all(ys, xs, ids, wts, W1, W2, f"swap step {step}")
        assert total_moves > 0, "the skewed routing never triggered a swap"
    finally:
        for l in layers:
            l.close()
        for rt in rts:
            rt.destroy()


def test_full_size_benchmark_step_sampled_against_oracle():
    """The benchmark's own configuration on one GPU (Qwen3-30B layer shape, all 128 experts, 512 tokens, top-8):
    a graph-launched step, checked against the CPU oracle on a sample of tokens (the oracle needs seconds per
    token batch at this size), plus exact conservation of the routed rows."""
    shape = wl.shape_of("qwen3-30b")
    S = 512
    cfg = EPMoEConfig(shape=shape, ranks=1, ranks_per_node=1, max_tokens_per_rank=S)
    _, _, ids, wts, _, _ = wl.make("qwen3-30b", 1)
    layer = EPMoE(cfg, LocalGroup(0, 1), ids, ids)
    wdev = wl.fast_weights(shape, range(shape.num_experts), torch.device("cuda"))
    layer.load_weights(lambda e: wdev[e][0], lambda e: wdev[e][1])
    x = wl.tokens(0, S, shape.hidden)
    y = layer.step(ids[0].cuda(), wts[0].cuda(), x.cuda()).clone()
    y_again = layer.step(ids[0].cuda(), wts[0].cuda(), x.cuda()).clone()
    layer.check()
    assert torch.equal(y, y_again)
    splits, m_this = layer.tables("splits", "m_this")
    assert int(splits.sum()) == S * shape.topk == int(m_this[0])
    sample = torch.arange(0, S, 16)
    W1 = torch.stack([wdev[e][0].cpu() for e in range(shape.num_experts)])
    W2 = torch.stack([wdev[e][1].cpu() for e in range(shape.num_experts)])
    _close(y[sample.cuda()], x[sample], ids[0][sample], wts[0][sample], W1, W2, "full-size sample")
    layer.close()


def test_trace_replay_batch_through_the_layer():
    """Routing drawn by the reference's batch sampler from a trace slice (here the committed synthetic slice),
    pool window for the placement: two emulated ranks, layer output and routed metadata against the oracle."""
    import os
    from zepp_b200 import traces
    data = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "traces")
    ts = traces.load_slice("qwen3", data)
    shape = ModelShape(ts.num_experts, ts.topk, 256, 128, act="swiglu")
    W, chunk, budget = 2, 256 * 2, 64 * 512 / (1 << 20)
    S = traces.tokens_per_rank(budget, chunk, ts.topk)
    assert S == 64
    ids = torch.tensor(traces.sample_batch(ts, W, W, budget, chunk), dtype=torch.int32).view(W, S, ts.topk)
    pool = torch.tensor(traces.pool_routing(ts, W, 256), dtype=torch.int32)
    gen = torch.Generator().manual_seed(5)
    wts = torch.softmax(torch.randn(W, S, ts.topk, generator=gen), dim=-1)
    cfg = EPMoEConfig(shape=shape, ranks=W, ranks_per_node=W, max_tokens_per_rank=S)
    layers, rts = make_local_layers(cfg, ids, pool, wait_limit_ms=500)
    W1, W2 = _weights(shape)
    try:
        for l in layers:
            l.load_weights(lambda e: W1[e], lambda e: W2[e])
        xs = [wl.tokens(r, S, shape.hidden, seed=3) for r in range(W)]
        ys = local_step(layers, [ids[r].cuda() for r in range(W)], [wts[r].cuda() for r in range(W)], [x.cuda() for x in xs])
        for l in layers:
            l.check()
        _check_all(ys, xs, ids, wts, W1, W2, "trace replay")
        pl0 = layers[0].placement
        pl = op.Placement(pl0.p2l.numpy(), pl0.l2p.numpy(), pl0.lcnts.numpy())
        phys, _ = op.reference_route(ids.numpy(), pl, cfg.slots_per_rank, W, cfg.router_c)
        vce = op.virtual_route(phys.reshape(W * S, -1), cfg.slots_per_rank, cfg.groups_per_rank)
        splits, scat, _, _ = op.routed_meta(vce, W, S, cfg.groups_per_rank, 1, W)
        assert np.array_equal(layers[1].tables("splits")[0].cpu().numpy(), splits)
        assert np.array_equal(layers[1].tables("scatter_index")[0].cpu().numpy().reshape(scat.shape), scat)
    finally:
        for l in layers:
            l.close()
        for rt in rts:
            rt.destroy()
