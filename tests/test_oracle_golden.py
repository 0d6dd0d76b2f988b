"""The CPU oracle (oracle/planner.py) against golden vectors produced by the reference's own
Python planner (tests/golden/make_golden.py).  Everything is integer work: bit-exact."""
import numpy as np

from oracle import planner as op


def _placement(c):
    return op.Placement(c["p2l"], c["l2p"], c["lcnts"])


def test_placement_matches_reference(planner_cases):
    for i in range(planner_cases.n):
        c = planner_cases.case(i)
        R, L, G, K, S, nlp, _, _ = [int(v) for v in c["dims"]]
        pl = op.solve_placement(op.demand_histogram(c["pool"], L, G), L, nlp)
        assert np.array_equal(pl.p2l, c["p2l"]), i
        assert np.array_equal(pl.l2p, c["l2p"]), i
        assert np.array_equal(pl.lcnts, c["lcnts"]), i


def test_route_tables_budgets_assignment(planner_cases):
    for i in range(planner_cases.n):
        c = planner_cases.case(i)
        R, L, G, K, S, nlp, c_num, c_den = [int(v) for v in c["dims"]]
        assert op.c_rational(c_num / c_den) == (c_num, c_den)
        phys, info = op.reference_route(c["topk"], _placement(c), nlp, L, c_num / c_den)
        tab = info["tables"]
        for name in ("M", "fill", "U", "Lb", "rep"):
            assert np.array_equal(tab[name], c[name]), (i, name)
        assert np.array_equal(info["release"], c["release"]), i
        assert np.array_equal(info["extra"], c["extra"]), i
        assert np.array_equal(info["phys0"], c["phys0"]), i
        assert np.array_equal(phys, c["phys"]), i


def test_meta_demands_capacities_plans(planner_cases):
    for i in range(planner_cases.n):
        c = planner_cases.case(i)
        R, L, G, K, S, nlp, c_num, c_den = [int(v) for v in c["dims"]]
        gpe, NN = nlp + 1, R // L
        vce = op.virtual_route(c["phys"].reshape(R * S, K), nlp, gpe)
        assert np.array_equal(vce, c["vce"]), i
        splits, scat, sps, uc = op.routed_meta(vce, R, S, gpe, NN, L)
        assert np.array_equal(splits, c["splits"]) and np.array_equal(scat, c["scatter"]), i
        assert np.array_equal(sps, c["sps"]) and np.array_equal(uc, c["uc"]), i
        assert op.demands_from_meta(sps, uc, R, L, gpe) == c["demands"].tolist(), i
        caps = op.compute_capacities(c["topk"], [_placement(c)], nlp, L, c_num / c_den)
        assert caps == c["caps"].tolist(), (i, caps, c["caps"].tolist())
        for r in range(R):
            words, head = op.dispatch_plan_head(sps, uc, R, L, gpe, r, S * K, 1 << 40)
            assert words[:head] == c["dplan_head"][r].tolist(), (i, r)
            if NN == 1:
                so, sr, do, lo = op.combine_tables(sps, R, gpe, r)
                assert np.concatenate([so, sr, do, lo]).tolist() == c["cplan"][r].tolist(), (i, r)


def test_violation_mask_bits():
    dem = [10, 11, 12, 13, 14, 15, 16]
    loose = [1 << 40] * 8
    assert op.violation_mask(dem, loose, False) == 0
    tight = [dem[0] - 1, dem[1] - 1, dem[2] - 1, dem[3] - 1, dem[0] - 1, dem[4] - 1, dem[5] - 1, dem[6] - 1]
    assert op.violation_mask(dem, tight, False) == 0x7F        # tests/test_meta_device.py:43-46
    assert op.violation_mask(dem, tight, True) == 0x81         # tests/test_meta_device.py:47-48


def test_swap_decision_sequences(swap_cases):
    nswaps = 0
    for i in range(swap_cases.n):
        s = swap_cases.case(i)
        R, L, G, nlp, steps = [int(v) for v in s["dims"]]
        for st in range(steps):
            p2l = s[f"p2l_in{st}"]
            pl = op.Placement(p2l, op.rebuild_l2p(p2l, G, R), s["lcnts"])
            load_g = s[f"loads{st}"].astype(np.int64).sum(0)
            new, rounds = op.decide_swaps(load_g, pl, L, nlp, 0.25)
            assert rounds == int(s[f"rounds{st}"][0]), (i, st)
            if rounds:
                nswaps += 1
                assert np.array_equal(new, s[f"p2l_out{st}"]), (i, st)
                assert np.array_equal(op.rebuild_l2p(new, G, R), s[f"l2p_out{st}"]), (i, st)
                mv = op.net_moves(p2l, new, L, nlp)
                flat = [(r,) + tuple(m) for r in range(R) for m in mv[r]]
                assert flat == [tuple(int(v) for v in row) for row in s[f"moves{st}"]], (i, st)
                blk = op.swap_result_block(load_g, pl, L, nlp, 0.25)
                assert blk[0] == rounds and blk[1] == len(flat)
            else:
                assert new is None
    assert nswaps >= 5


def test_benchmark_config_expectations(config_cases):
    """Full-size seeded benchmark routings: rows per rank, capacities and the step-0 swap verdict."""
    z = config_cases
    for name in ("qwen30b_w8", "qwen235b_w2", "qwen235b_w4", "qwen235b_w8", "qwen235b_w8_l4"):
        W, L, G, K, S, nlp, _, _ = [int(v) for v in z[f"{name}.dims"]]
        topk = z[f"{name}.topk"].astype(np.int64)
        pl = op.solve_placement(op.demand_histogram(topk, L, G), L, nlp)
        assert np.array_equal(pl.p2l, z[f"{name}.p2l"]), name
        phys, _ = op.reference_route(topk, pl, nlp, L, 0.25)
        assert np.array_equal(phys, z[f"{name}.phys"].astype(np.int32)), name
        gpe = nlp + 1
        splits, scat, sps, uc = op.routed_meta(op.virtual_route(phys.reshape(W * S, K), nlp, gpe), W, S, gpe, W // L, L)
        assert np.array_equal(splits, z[f"{name}.splits"]), name
        assert np.array_equal(uc, z[f"{name}.uc"]), name
        m_r = sps.astype(np.int64).reshape(W, W, gpe).sum(2).sum(0)
        assert m_r.tolist() == z[f"{name}.m_r"].tolist(), name
        chk = int((scat.astype(np.int64).reshape(-1) * np.arange(1, scat.size + 1)).sum())
        assert chk == int(z[f"{name}.scatter_sum"][0]), name
        load_g = np.bincount(topk.reshape(-1), minlength=G)
        new, rounds = op.decide_swaps(load_g, pl, L, nlp, 0.25)
        assert rounds == int(z[f"{name}.swap"][0]), name
        if rounds:
            assert np.array_equal(new, z[f"{name}.p2l_swapped"]), name
            assert sum(len(m) for m in op.net_moves(pl.p2l, new, L, nlp)) == int(z[f"{name}.swap"][1])
