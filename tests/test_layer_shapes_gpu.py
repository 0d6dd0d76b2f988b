"""Layer-output parity on the benchmark's own layer shapes (Qwen3-235B-A22B: H=4096, I=1536, E=128; Kimi-K2:
H=7168, I=2048, E=384), on token buckets from 8 to 4096 rows, on steps with pad rows, and the give-up path of a
device-side wait.  Weights are generated per expert on the device (workloads.device_expert); the CPU oracle
regenerates only the experts that a sample of tokens touches, so these sizes stay within seconds on the host.
Planner products are compared exactly on the full routing."""
import numpy as np
import pytest
import torch

from oracle import planner as op
from zepp_b200 import EPMoE, EPMoEConfig, ModelShape
from zepp_b200 import workloads as wl
from zepp_b200.layer import LocalGroup, local_step, make_local_layers, token_buckets

from test_layer_gpu import _close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _touched(shape, ids_sample):
    """{expert: cpu weights} of the experts a token sample picks (device_expert is a function of the id)."""
    experts = sorted({int(e) for e in ids_sample.reshape(-1).tolist() if e >= 0})
    W1, W2 = {}, {}
    for e in experts:
        w1, w2 = wl.device_expert(e, shape, torch.device(DEV))
        W1[e], W2[e] = w1.cpu(), w2.cpu()
    return W1, W2


def _planner_exact(layers, ids, cfg, W, L, S):
    """Every rank's routed metadata equals the oracle's on the whole routing."""
    pl0 = layers[0].placement
    pl = op.Placement(pl0.p2l.numpy(), pl0.l2p.numpy(), pl0.lcnts.numpy())
    phys, _ = op.reference_route(ids.numpy(), pl, cfg.slots_per_rank, L, cfg.router_c)
    vce = op.virtual_route(phys.reshape(W * S, -1), cfg.slots_per_rank, cfg.groups_per_rank)
    splits, scat, sps, uc = op.routed_meta(vce, W, S, cfg.groups_per_rank, W // L, L)
    gpe = cfg.groups_per_rank
    for r, l in enumerate(layers):
        t = dict(zip(("vce", "splits", "scatter_index", "sps", "uc", "m_this"),
                     l.tables("vce", "splits", "scatter_index", "sps", "uc", "m_this")))
        assert np.array_equal(t["vce"].cpu().numpy().reshape(vce.shape), vce), (r, "vce")
        assert np.array_equal(t["splits"].cpu().numpy(), splits), (r, "splits")
        assert np.array_equal(t["scatter_index"].cpu().numpy().reshape(scat.shape), scat), (r, "scatter")
        assert np.array_equal(t["sps"].cpu().numpy().reshape(sps.shape), sps), (r, "sps")
        assert np.array_equal(t["uc"].cpu().numpy().reshape(uc.shape), uc), (r, "uc")
        assert int(t["m_this"][0]) == int(splits[r * gpe:(r + 1) * gpe].sum())


@pytest.mark.parametrize("name,zipf,strategy", [("qwen3-235b", 1.0, "overlap"), ("k2", 1.2, "overlap"),
                                                ("qwen3-235b", 1.0, "direct")])
def test_benchmark_shapes_eight_emulated_ranks(name, zipf, strategy):
    """Full H, I and E of the 235B and K2 layer shapes, sharded 8 ways on one GPU, 64 tokens per rank (K2: 51
    groups per rank, 408 virtual experts: the metadata kernels' large shared-memory configuration)."""
    shape = wl.shape_of(name)
    W, S = 8, 64
    cfg = EPMoEConfig(shape=shape, ranks=W, ranks_per_node=W, max_tokens_per_rank=S, comm_strategy=strategy)
    gen = torch.Generator().manual_seed(1)
    ids, wts = wl.routing(W, S, shape.topk, wl.popularity(shape.num_experts, zipf, gen), gen)
    layers, rts = make_local_layers(cfg, ids, ids, wait_limit_ms=2000)
    dev = torch.device(DEV)
    try:
        for l in layers:
            l.load_weights(lambda e: wl.device_expert(e, shape, dev)[0], lambda e: wl.device_expert(e, shape, dev)[1])
        xs = [wl.tokens(r, S, shape.hidden, seed=3) for r in range(W)]
        ys = local_step(layers, [ids[r].cuda() for r in range(W)], [wts[r].cuda() for r in range(W)],
                        [x.cuda() for x in xs])
        for l in layers:
            l.check()
        _planner_exact(layers, ids, cfg, W, W, S)
        for r, toks in ((0, [0, 33]), (5, [7]), (7, [63])):          # a few tokens of three ranks: ~30 experts
            t = torch.tensor(toks)
            W1, W2 = _touched(shape, ids[r][t])
            _close(ys[r][t.cuda()], xs[r][t], ids[r][t], wts[r][t], W1, W2, f"{name} {strategy} rank{r}")
        splits = layers[0].tables("splits")[0]
        assert int(splits.sum()) == W * S * shape.topk
    finally:
        for l in layers:
            l.close()
        for rt in rts:
            rt.destroy()


def test_full_size_235b_buckets_on_one_gpu():
    """The Qwen3-235B layer on one GPU (all 128 experts, 4.8 GB of weights), Zipf 1.0 routing, one layer sized for
    4096 tokens stepping through the buckets 8 ... 4096 (graph-launched steps): sampled tokens against the oracle,
    exact row conservation, and bitwise repeatability of a bucket revisited."""
    shape = wl.shape_of("qwen3-235b")
    S_max = 4096
    cfg = EPMoEConfig(shape=shape, ranks=1, ranks_per_node=1, max_tokens_per_rank=S_max)
    assert token_buckets(cfg) == [8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096]
    gen = torch.Generator().manual_seed(0)
    p = wl.popularity(shape.num_experts, 1.0, gen)
    ids_all, wts_all = wl.routing(1, S_max, shape.topk, p, gen)
    layer = EPMoE(cfg, LocalGroup(0, 1), ids_all, ids_all)
    dev = torch.device(DEV)
    layer.load_weights(lambda e: wl.device_expert(e, shape, dev)[0], lambda e: wl.device_expert(e, shape, dev)[1])
    x_all = wl.tokens(0, S_max, shape.hidden)
    first = {}
    try:
        for S in (512, 8, 32, 128, 2048, 4096, 8):
            layer.set_tokens(S)
            ids, wts, x = ids_all[0, :S].contiguous(), wts_all[0, :S].contiguous(), x_all[:S].contiguous()
            y = layer.step(ids.cuda(), wts.cuda(), x.cuda()).clone()
            layer.check()
            splits, m_this = layer.tables("splits", "m_this")
            assert int(splits.sum()) == S * shape.topk == int(m_this[0]), S
            if S in first:
                assert torch.equal(first[S], y), f"bucket {S} revisited gave different bits"
                continue
            first[S] = y
            t = torch.tensor(sorted({0, S // 2, S - 1}))
            W1, W2 = _touched(shape, ids[t])
            _close(y[t.cuda()], x[t], ids[t], wts[t], W1, W2, f"235b W=1 S={S}")
    finally:
        layer.close()


def test_pad_rows_cost_nothing_and_change_nothing():
    """A step of n real tokens padded to its bucket (expert id -1 on the pad rows): real rows equal the oracle,
    pad copies are counted in no split / load / unique count and get scatter_index -1, on one rank and on four
    emulated ranks with a different number of real tokens each."""
    shape = ModelShape(32, 8, 512, 256, act="swiglu")
    W1 = torch.stack([wl.expert_w1(e, shape) for e in range(shape.num_experts)])
    W2 = torch.stack([wl.expert_w2(e, shape) for e in range(shape.num_experts)])
    # ---- one rank, step_padded picks the bucket
    cfg = EPMoEConfig(shape=shape, ranks=1, ranks_per_node=1, max_tokens_per_rank=64)
    gen = torch.Generator().manual_seed(2)
    p = wl.popularity(shape.num_experts, 1.0, gen)
    ids, wts = wl.routing(1, 64, shape.topk, p, gen)
    layer = EPMoE(cfg, LocalGroup(0, 1), ids, ids)
    layer.load_weights(lambda e: W1[e], lambda e: W2[e])
    x = wl.tokens(0, 64, shape.hidden)
    try:
        for n in (1, 5, 8, 19, 64, 1):
            y = layer.step_padded(ids[0, :n].cuda(), wts[0, :n].cuda(), x[:n].cuda())
            layer.check()
            assert y.shape[0] == n
            _close(y, x[:n], ids[0, :n], wts[0, :n], W1, W2, f"padded n={n}")
            bucket = next(b for b in token_buckets(cfg) if b >= n)
            splits, scat, vce = layer.tables("splits", "scatter_index", "vce")
            assert int(splits.sum()) == n * shape.topk
            scat = scat.cpu().numpy().reshape(bucket, shape.topk)
            assert (scat[:n] >= 0).all() and (scat[n:] == -1).all() and (vce.cpu().numpy().reshape(bucket, -1)[n:] == -1).all()
    finally:
        layer.close()
    # ---- four emulated ranks with ragged real counts inside a bucket of 16
    W, S = 4, 16
    cfg = EPMoEConfig(shape=shape, ranks=W, ranks_per_node=W, max_tokens_per_rank=S)
    ids, wts = wl.routing(W, S, shape.topk, p, gen)
    counts = [16, 3, 0, 9]
    for r, n in enumerate(counts):
        ids[r, n:] = -1
        wts[r, n:] = 0
    sizing = ids.clamp_min(0)
    layers, rts = make_local_layers(cfg, sizing, sizing, wait_limit_ms=1000)
    try:
        for l in layers:
            l.load_weights(lambda e: W1[e], lambda e: W2[e])
        xs = [wl.tokens(r, S, shape.hidden, seed=9) for r in range(W)]
        for strategy_step in range(2):
            ys = local_step(layers, [ids[r].cuda() for r in range(W)], [wts[r].cuda() for r in range(W)],
                            [x.cuda() for x in xs])
            for l in layers:
                l.check()
        pl = layers[0].placement
        assert int(pl.lcnts.max()) == 1
        slot = pl.l2p[:, 0].numpy()
        phys = np.where(ids.numpy() >= 0, slot[ids.clamp_min(0).numpy()], -1)
        nlp, gpe = cfg.slots_per_rank, cfg.groups_per_rank
        vce = np.where(phys >= 0, (phys // nlp) * gpe + 1 + phys % nlp, -1).reshape(W * S, -1)
        splits, scat, sps, uc = op.routed_meta(vce, W, S, gpe, 1, W)
        for r, l in enumerate(layers):
            t = dict(zip(("vce", "splits", "scatter_index", "sps", "uc"), l.tables("vce", "splits", "scatter_index", "sps", "uc")))
            assert np.array_equal(t["vce"].cpu().numpy().reshape(vce.shape), vce), r
            assert np.array_equal(t["splits"].cpu().numpy(), splits), r
            assert np.array_equal(t["scatter_index"].cpu().numpy().reshape(scat.shape), scat), r
            assert np.array_equal(t["sps"].cpu().numpy().reshape(sps.shape), sps), r
            assert np.array_equal(t["uc"].cpu().numpy().reshape(uc.shape), uc), r
            n = counts[r]
            if n:
                _close(ys[r][:n], xs[r][:n], ids[r, :n], wts[r, :n], W1, W2, f"ragged rank{r}")
        assert int(splits.sum()) == sum(counts) * shape.topk
    finally:
        for l in layers:
            l.close()
        for rt in rts:
            rt.destroy()


def test_a_wait_that_runs_out_is_reported_and_the_next_layer_works():
    """Two emulated ranks; rank 1 never pushes its token rows, so rank 0's dispatch GEMM waits for a flag that
    nothing raises.  The wait is bounded (50 ms here): the kernel records what it waited for, frees its tensor
    memory and returns, check() raises, and a fresh layer on the same context passes afterwards."""
    shape = ModelShape(32, 8, 512, 256, act="swiglu")
    W, S = 2, 64
    cfg = EPMoEConfig(shape=shape, ranks=W, ranks_per_node=W, max_tokens_per_rank=S)
    gen = torch.Generator().manual_seed(6)
    ids, wts = wl.routing(W, S, shape.topk, wl.popularity(shape.num_experts, 0.0, gen), gen)
    W1 = torch.stack([wl.expert_w1(e, shape) for e in range(shape.num_experts)])
    W2 = torch.stack([wl.expert_w2(e, shape) for e in range(shape.num_experts)])
    layers, rts = make_local_layers(cfg, ids, ids, wait_limit_ms=50)
    xs = [wl.tokens(r, S, shape.hidden) for r in range(W)]
    try:
        for l in layers:
            l.load_weights(lambda e: W1[e], lambda e: W2[e])
        for ph in range(4):
            for r, l in enumerate(layers):
                l.prepare(ids[r].cuda(), wts[r].cuda(), phase=ph)
        layers[0].forward(xs[0].cuda(), phase=0)          # rank 0 pushes; rank 1 does not
        layers[0].forward(xs[0].cuda(), phase=1)          # its dispatch GEMM gives up on rank 1's rows
        with pytest.raises(RuntimeError, match="a device-side wait ran out") as ei:
            layers[0].check()
        assert "wait id 3" in str(ei.value) or "wait id 9" in str(ei.value), str(ei.value)   # the x flag, or a tile that never filled
        assert float(torch.ones(4, device="cuda").sum()) == 4.0
    finally:
        for l in layers:
            l.close()
        for rt in rts:
            rt.destroy()
    layers, rts = make_local_layers(cfg, ids, ids, wait_limit_ms=500)
    try:
        for l in layers:
            l.load_weights(lambda e: W1[e], lambda e: W2[e])
        ys = local_step(layers, [ids[r].cuda() for r in range(W)], [wts[r].cuda() for r in range(W)],
                        [x.cuda() for x in xs])
        for r, l in enumerate(layers):
            l.check()
            _close(ys[r], xs[r], ids[r], wts[r], W1, W2, f"after the timeout rank{r}")
    finally:
        for l in layers:
            l.close()
        for rt in rts:
            rt.destroy()
