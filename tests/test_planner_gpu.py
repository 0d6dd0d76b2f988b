"""The CUDA planner through the C-ABI against the CPU oracle and the golden vectors of the
reference's planner.  Integer work: everything must be bit-exact.  One GPU plays every rank, as
the reference's device tests do (tests/test_route_fused.py:72-79)."""
import numpy as np
import pytest
import torch

from oracle import planner as op
from zepp_b200._ext import C

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _dev(a, dt=torch.int32):
    return torch.as_tensor(np.ascontiguousarray(a)).to(device=DEV, dtype=dt).contiguous()


def _ws_tables(ws, G, R):
    off = C.route_ws_offsets(G, R)
    CM = min(R, 32)
    w = ws.cpu().numpy().astype(np.int64)
    g = lambda k, n: w[off[k]:off[k] + n]  # noqa: E731
    return dict(rep=g("rep", G * CM).reshape(G, CM), c=g("c", G), D=g("D", G), U=g("U", G), Lb=g("Lb", G),
                fill=g("fill", G * CM).reshape(G, CM), M=g("M", G * R * CM).reshape(G, R, CM),
                release=g("release", G * CM).reshape(G, CM), extra=g("extra", G * CM).reshape(G, CM)), CM


def test_route_against_golden(planner_cases):
    """tables, bounds, budgets (before the vacate pass), water-fill assignment and vacated
    assignment of every rank == the reference planner's (python/zepp/routing.py)."""
    for i in range(planner_cases.n):
        c = planner_cases.case(i)
        R, L, G, K, S, nlp, c_num, c_den = [int(v) for v in c["dims"]]
        topk = _dev(c["topk"])
        loads = torch.stack([torch.bincount(topk[r].reshape(-1).long(), minlength=G) for r in range(R)]).int().contiguous()
        l2p, lcnts = _dev(c["l2p"]), _dev(c["lcnts"])
        Cmax = c["M"].shape[2]
        for r in range(R):
            ws = torch.full((C.route_workspace_ints(G, R),), -7, dtype=torch.int32, device=DEV)
            C.route_tables_only(loads, l2p, lcnts, r, nlp, L, c_num, c_den, ws)
            tab, CM = _ws_tables(ws, G, R)
            assert np.array_equal(tab["M"][:, :, :Cmax], c["M"]), (i, r, "M")
            assert np.array_equal(tab["fill"][:, :Cmax], c["fill"]), (i, r, "fill")
            assert np.array_equal(tab["U"], c["U"]) and np.array_equal(tab["Lb"], c["Lb"]), (i, r, "bounds")
            assert np.array_equal(tab["rep"][:, :Cmax], c["rep"]), (i, r, "rep")
            assert np.array_equal(tab["release"][:, :Cmax], c["release"][:, r, :]), (i, r, "release")
            assert np.array_equal(tab["extra"][:, :Cmax], c["extra"][:, r, :]), (i, r, "extra")
            probs = torch.rand(S, K, device=DEV)
            send = torch.full((2 * S * K,), -7, dtype=torch.int32, device=DEV)
            phys, stats = C.route_fused(topk[r], loads, l2p, lcnts, r, nlp, L, c_num, c_den, ws, probs.view(-1), send)
            assert np.array_equal(phys.cpu().numpy(), c["phys"][r]), (i, r, "phys")
            st = stats.cpu().tolist()
            assert st[0] == 0 and st[2] == 0, (i, r, st)
            assert torch.equal(send[:S * K], phys.reshape(-1))
            assert torch.equal(send[S * K:], probs.view(-1).view(torch.int32))
            # release + extra per replica is invariant under the vacate pass (tests/test_route_fused.py:84-89)
            tab2, _ = _ws_tables(ws, G, R)
            assert np.array_equal((tab2["release"] + tab2["extra"])[:, :Cmax],
                                  c["release"][:, r, :] + c["extra"][:, r, :]), (i, r)


def _check_meta(vce, W, L, gpe, tag, gold=None):
    S = vce.shape[0] // W
    K = vce.shape[1]
    NN = W // L
    ref = op.routed_meta(vce, W, S, gpe, NN, L)
    dem_ref = op.demands_from_meta(ref[2], ref[3], W, L, gpe)
    for rank in sorted({0, W // 2, W - 1}):
        o = C.routed_meta_full(W, L, S, K, gpe - 1, gpe, vce=_dev(vce), my_rank=rank)
        for name, r in zip(("splits", "scatter_index", "sps", "uc"), ref):
            assert np.array_equal(o[name].cpu().numpy().reshape(r.shape), r), (tag, name)
        dd = o["demands"].cpu().tolist()
        assert dd[:7] == dem_ref and dd[7] == 0, (tag, dd, dem_ref)
        words, head = op.dispatch_plan_head(ref[2], ref[3], W, L, gpe, rank, S * K, 1 << 40)
        assert o["dplan"].cpu().tolist()[:head] == words[:head], (tag, rank, "dplan")
        if NN == 1:
            so, sr, do, lo = op.combine_tables(ref[2], W, gpe, rank)
            assert o["cplan"].cpu().tolist() == np.concatenate([so, sr, do, lo]).tolist(), (tag, rank, "cplan")
    # every capacity one short of its demand raises every bit; direct: bits 0 and 7 (tests/test_meta_device.py:43-48)
    d = dem_ref
    tight = [d[0] - 1, d[1] - 1, d[2] - 1, d[3] - 1, d[0] - 1, d[4] - 1, d[5] - 1, d[6] - 1]
    o = C.routed_meta_full(W, L, S, K, gpe - 1, gpe, vce=_dev(vce), caps=tight)
    assert int(o["demands"][7]) == 0x7F, (tag, o["demands"].tolist())
    o = C.routed_meta_full(W, L, S, K, gpe - 1, gpe, vce=_dev(vce), caps=tight, direct=True)
    assert int(o["demands"][7]) == 0x81, tag
    # tight receive / send capacities raise the plan's error bits (tests/test_dispatch_plan_device.py:39-48)
    o = C.routed_meta_full(W, L, S, K, gpe - 1, gpe, vce=_dev(vce), caps=[0] * 8, copies_per_rank=0)
    if int(ref[3].sum()) > 0:
        assert int(o["dplan"][5]) & 48 == 48, tag
    return ref


def test_meta_against_golden_and_oracle(planner_cases):
    for i in range(planner_cases.n):
        c = planner_cases.case(i)
        R, L, G, K, S, nlp, _, _ = [int(v) for v in c["dims"]]
        ref = _check_meta(c["vce"], R, L, nlp + 1, f"golden{i}")
        for name, r in zip(("splits", "scatter", "sps", "uc"), ref):
            assert np.array_equal(r.reshape(c[name].shape), c[name]), (i, name)


def test_meta_shape_grid_and_adversarial():
    """Shape grid of the reference's metadata test (tests/test_meta_device.py:58-75): K = 8 and 6,
    several tiles per source, skewed / one-expert / two-expert routings, duplicate picks in a token."""
    rng = np.random.default_rng(1)
    for W, L in ((4, 4), (8, 8), (8, 4), (16, 4)):
        for S in (8, 136, 264):
            for gpe in (5, 11):
                nlp = gpe - 1
                for K in (8, 6):
                    if K == 6 and S != 136:
                        continue
                    phys = rng.integers(0, W * nlp, size=(W * S, K))
                    _check_meta(op.virtual_route(phys, nlp, gpe), W, L, gpe, f"random W{W} S{S} K{K} gpe{gpe}")
                phys = rng.integers(0, nlp, size=(W * S, 8))          # everything on rank 0, duplicates
                _check_meta(op.virtual_route(phys, nlp, gpe), W, L, gpe, f"skewed W{W} S{S}")
            E = W * 5
            _check_meta(np.full((W * S, 8), 1, dtype=np.int32), W, L, 5, f"one-expert W{W} S{S}")
            two = (rng.integers(0, 2, size=(W * S, 8)) * (E - 1)).astype(np.int32)
            _check_meta(two, W, L, 5, f"two-experts W{W} S{S}")


def test_planner_tail_from_gathered_rows():
    """gathered [R, 2n] (phys | weight bits) -> vce, probs_all (src/planner/lane_device.cu:526-540)."""
    R, L, S, K, nlp = 4, 4, 40, 8, 6
    gpe = nlp + 1
    g = torch.Generator().manual_seed(5)
    phys = torch.randint(0, R * nlp, (R, S * K), generator=g, dtype=torch.int32)
    w = torch.rand(R, S * K, generator=g)
    gathered = torch.cat([phys, w.view(torch.int32)], dim=1).contiguous().to(DEV)
    o = C.routed_meta_full(R, L, S, K, nlp, gpe, gathered=gathered)
    assert np.array_equal(o["vce"].cpu().numpy().reshape(-1), op.virtual_route(phys.numpy().reshape(-1), nlp, gpe))
    assert torch.equal(o["probs_all"].cpu().view(R, S * K), w)


def test_swap_decide_and_lane_arm(swap_cases):
    """Device decision == host decision on the golden sequences: trigger, new p2l / l2p, per-rank pull
    lists, result block; lane_arm == tests/test_lane_device.py:36-58."""
    cap = 8
    swaps = 0
    for i in range(swap_cases.n):
        s = swap_cases.case(i)
        R, L, G, nlp, steps = [int(v) for v in s["dims"]]
        for st in range(steps):
            p2l_in = s[f"p2l_in{st}"]
            loads = s[f"loads{st}"]
            pl = op.Placement(p2l_in, op.rebuild_l2p(p2l_in, G, R), s["lcnts"])
            blk_ref = op.swap_result_block(loads.astype(np.int64).sum(0), pl, L, nlp, 0.25)
            p2l, l2p = _dev(p2l_in), _dev(pl.l2p)
            out = torch.zeros(C.swap_decide_out_ints(R, G, nlp, cap), dtype=torch.int64, device=DEV)
            C.swap_decide(_dev(loads), p2l, l2p, _dev(s["lcnts"]), L, nlp, 0.25, cap, 32, out)
            blk = out.cpu().numpy()
            assert np.array_equal(blk, blk_ref), (i, st, np.nonzero(blk != blk_ref)[0][:8])
            rounds = int(s[f"rounds{st}"][0])
            assert int(blk[0]) == rounds
            if rounds:
                swaps += 1
                assert np.array_equal(p2l.cpu().numpy(), s[f"p2l_out{st}"]), (i, st)
                assert np.array_equal(l2p.cpu().numpy(), s[f"l2p_out{st}"]), (i, st)
            else:
                assert np.array_equal(p2l.cpu().numpy(), p2l_in) and np.array_equal(l2p.cpu().numpy(), pl.l2p)
            moves = op.net_moves(p2l_in, blk_ref[3 + R + 4 * R * cap:3 + R + 4 * R * cap + R * nlp], L, nlp) \
                if rounds else [[] for _ in range(R)]
            stag = [[(k + 1) * 10 ** 9 + j * 4096 for j in range(cap)] for k in (0, 1)]
            for r in range(R):
                gpe = nlp + 1
                gate = torch.full((2 * gpe,), -7, dtype=torch.int64, device=DEV)
                sched = torch.full((gpe,), -7, dtype=torch.int32, device=DEV)
                ovr = [torch.full((gpe,), -7, dtype=torch.int64, device=DEV) for _ in (0, 1)]
                C.lane_arm(out, R, r, nlp, cap, gate, sched, ovr[0], ovr[1],
                           torch.tensor(stag, dtype=torch.int64, device=DEV), 1000 + st)
                eg, es, eo = op.lane_arm_expect(moves[r], nlp, 1000 + st, stag)
                assert np.array_equal(gate.cpu().numpy(), eg), (i, st, r, "gate")
                assert np.array_equal(sched.cpu().numpy(), es), (i, st, r, "sched")
                assert np.array_equal(ovr[0].cpu().numpy(), eo[0]) and np.array_equal(ovr[1].cpu().numpy(), eo[1])
    assert swaps >= 5


def test_bounded_wait_gives_up_and_context_survives():
    """A wait on a flag nobody raises returns 'gave up' after its limit; the context stays usable."""
    flag = torch.zeros(1, dtype=torch.int64, device=DEV)
    res = C.wait_geq(flag, 5, 20)
    torch.cuda.synchronize()
    assert int(res[0]) == 0
    flag.fill_(7)
    res = C.wait_geq(flag, 5, 20)
    assert int(res[0]) == 1
    assert float(torch.ones(4, device=DEV).sum()) == 4.0


def test_capacities_against_golden(planner_cases, config_cases):
    """Init-time capacity sizing through the device router == the reference's compute_capacities
    (python/zepp/routing.py:400-458), on the small golden cases and on the full-size benchmark
    routings including their swap orbits."""
    from zepp_b200.placement import Placement
    from zepp_b200.routing import compute_capacities
    from zepp_b200.swap import swap_orbit
    for i in range(0, planner_cases.n, 3):
        c = planner_cases.case(i)
        R, L, G, K, S, nlp, c_num, c_den = [int(v) for v in c["dims"]]
        pl = Placement(torch.from_numpy(c["p2l"]), torch.from_numpy(c["l2p"]), torch.from_numpy(c["lcnts"]), {})
        caps = compute_capacities(torch.from_numpy(c["topk"]), [pl], nlp, L, c_num / c_den, None)
        assert caps.as_list() == c["caps"].tolist(), (i, caps.as_list(), c["caps"].tolist())
    z = config_cases
    for name in ("qwen30b_w8", "qwen235b_w4", "qwen235b_w8", "qwen235b_w8_l4", "k2_w8"):
        W, L, G, K, S, nlp, zs, _ = [int(v) for v in z[f"{name}.dims"]]
        topk = torch.from_numpy(z[f"{name}.topk"].astype(np.int32))
        p2l = torch.from_numpy(z[f"{name}.p2l"])
        from zepp_b200.placement import rebuild_l2p
        lcnts = torch.bincount(p2l[p2l >= 0].long(), minlength=G).int()
        pl = Placement(p2l, rebuild_l2p(p2l, G, W), lcnts, {})
        placements = [pl]
        if zs:
            load_g = torch.bincount(topk.reshape(-1).long(), minlength=G)
            placements += swap_orbit(load_g, pl, L, nlp, 0.25)
        caps = compute_capacities(topk, placements, nlp, L, 0.25, None)
        assert caps.as_list() == z[f"{name}.caps"].tolist(), (name, caps.as_list(), z[f"{name}.caps"].tolist())
