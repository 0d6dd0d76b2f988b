"""Generates tests/golden/*.npz from the reference's own Python planner.

Run in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

The reference's `zepp` package imports a compiled NVSHMEM extension at import time; only its pure
Python planner is needed here, so `zepp._ext` is replaced by an empty stub before the import.
The fixtures are small seeded cases; the tests compare the oracle (oracle/planner.py) and the
CUDA planner against them bit for bit.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    ext = types.ModuleType("zepp._ext")
    ext.C = None
    ext.ensure_shm = lambda group: None
    sys.modules["zepp._ext"] = ext
    sys.path.insert(0, os.path.join(root, "python"))
    import zepp  # noqa: F401
    from zepp import capacity, placement, routing, swap
    return placement, routing, swap, capacity


def skewed(G, gen, hot=0.25, mass=0.7):
    perm = torch.randperm(G, generator=gen)
    p = torch.full((G,), (1 - mass) / (G - int(G * hot)))
    p[perm[:int(G * hot)]] = mass / int(G * hot)
    return p


def zipf(G, s, gen):
    perm = torch.randperm(G, generator=gen)
    p = torch.empty(G)
    p[perm] = (torch.arange(G, dtype=torch.float64) + 1.0).pow(-s).float()
    return p / p.sum()


def sample(p, n, K, gen):
    return torch.multinomial(p.expand(n, -1), K, replacement=False, generator=gen).int()


def npi(t, dt=np.int32):
    return np.asarray(t.cpu().numpy() if hasattr(t, "cpu") else t).astype(dt)


def route_case(mods, R, L, G, K, S, nlp, C, gen, shift):
    placement, routing, swap, capacity = mods
    p = skewed(G, gen)
    pool = torch.multinomial(p, R * 256 * K, replacement=True, generator=gen).view(R, 256, K).int()
    pl = placement.solve_placement(placement.demand_histogram(pool, L, G), L, nlp)
    if shift:
        p = skewed(G, gen)
    topk = sample(p, R * S, K, gen).view(R, S, K)
    c_num, c_den = routing.c_rational(C)
    phys0, tab = routing.route_water_fill(topk, pl.p2l, pl.l2p, pl.lcnts, nlp, L, c_num, c_den)
    phys, info = routing.reference_route(topk, pl, nlp, L, C)
    gpe = nlp + 1
    NN = R // L
    vce = routing.virtual_route(phys.view(R * S, K), nlp, gpe)
    splits, scat, sps, uc = routing.meta_from_virtual_route(vce, R, S, gpe, NN, L)
    dem = capacity.demands_from_meta(sps.numpy(), uc.numpy(), R, L, gpe)
    caps = routing.compute_capacities(topk, [pl], nlp, L, C)
    out = dict(
        dims=np.array([R, L, G, K, S, nlp, c_num, c_den], dtype=np.int64),
        pool=npi(pool), topk=npi(topk), p2l=npi(pl.p2l), l2p=npi(pl.l2p), lcnts=npi(pl.lcnts),
        M=npi(tab["M"], np.int64), fill=npi(tab["fill"], np.int64), U=npi(tab["U"], np.int64),
        Lb=npi(tab["Lb"], np.int64), rep=npi(tab["rep"], np.int64),
        release=npi(info["release"], np.int64), extra=npi(info["extra"], np.int64),
        phys0=npi(phys0), phys=npi(phys), vce=npi(vce), splits=npi(splits), scatter=npi(scat),
        sps=npi(sps), uc=npi(uc),
        demands=np.array([dem.recv_rows, dem.dispatch_recv, dem.dispatch_stage, dem.dispatch_relay,
                          dem.combine_conv, dem.combine_wire, dem.pair_rows], dtype=np.int64),
        caps=np.array([caps.recv_cap, caps.dispatch_recv, caps.dispatch_stage, caps.dispatch_relay,
                       caps.combine_send, caps.combine_conv, caps.combine_wire, caps.pair_cap], dtype=np.int64),
    )
    lay = routing.dispatch_plan_layout(L, NN)
    head = lay["round0"] + 3 * L
    BIG = 1 << 40
    dplan = [routing.dispatch_plan_ref(sps.numpy(), uc.numpy(), R, L, gpe, r, 2, S * K, BIG, BIG, BIG)[:head]
             for r in range(R)]
    out["dplan_head"] = np.array(dplan, dtype=np.int64)
    clay = routing.combine_plan_layout(R, NN, gpe)
    if NN == 1:
        cp = []
        for r in range(R):
            blk, _ = routing.combine_plan_ref(sps.numpy(), uc.numpy(), R, gpe, L, NN, r)
            cp.append(np.concatenate([blk[clay["send_off"]:clay["send_off"] + R + 1],
                                      blk[clay["send_rows"]:clay["send_rows"] + R],
                                      blk[clay["dst_off"]:clay["dst_off"] + R],
                                      blk[clay["lane_off"]:clay["lane_off"] + R + 1]]))
        out["cplan"] = np.array(cp, dtype=np.int64)
    return out


def swap_sequence(mods, R, L, G, steps, gen, C=0.25):
    placement, routing, swap, capacity = mods
    K = 8
    nlp = G // R + 2
    p = skewed(G, gen)
    pool = torch.multinomial(p, R * 256 * K, replacement=True, generator=gen).view(R, 256, K).int()
    pl = placement.solve_placement(placement.demand_histogram(pool, L, G), L, nlp)
    rec = dict(dims=np.array([R, L, G, nlp, steps], dtype=np.int64), lcnts=npi(pl.lcnts))
    for st in range(steps):
        if st % 3 == 2:
            p = skewed(G, gen)
        loads = torch.stack([torch.bincount(torch.multinomial(p, 128 * K, replacement=True, generator=gen),
                                            minlength=G) for _ in range(R)]).int()
        load_g = loads.long().sum(0)
        new_pl, rounds = swap.decide_swaps(load_g, pl, L, nlp, C)
        rec[f"loads{st}"] = npi(loads)
        rec[f"p2l_in{st}"] = npi(pl.p2l)
        rec[f"rounds{st}"] = np.array([rounds], dtype=np.int64)
        if new_pl is not None:
            mv = swap.net_moves(pl.p2l, new_pl.p2l, L, nlp)
            rec[f"p2l_out{st}"] = npi(new_pl.p2l)
            rec[f"l2p_out{st}"] = npi(new_pl.l2p)
            flat = [(r,) + tuple(m) for r in range(R) for m in mv[r]]
            rec[f"moves{st}"] = np.array(flat, dtype=np.int64).reshape(-1, 5)
            pl = new_pl
    return rec


def config_case(mods, name, W, L, G, K, S, zipf_s, C, with_swap, seed=0):
    """Planner products of a full-size benchmark routing (summary numbers + digests only)."""
    placement, routing, swap, capacity = mods
    gen = torch.Generator().manual_seed(seed)
    p = torch.full((G,), 1.0 / G) if zipf_s == 0 else zipf(G, zipf_s, gen)
    topk = sample(p, W * S, K, gen).view(W, S, K)
    nlp = G // W + 2
    gpe = nlp + 1
    pl = placement.solve_placement(placement.demand_histogram(topk, L, G), L, nlp)
    placements = [pl]
    load_g = torch.bincount(topk.reshape(-1).long(), minlength=G)
    if with_swap:
        placements += swap.swap_orbit(load_g, pl, L, nlp, C)
    caps = routing.compute_capacities(topk, placements, nlp, L, C)
    phys, _ = routing.reference_route(topk, pl, nlp, L, C)
    vce = routing.virtual_route(phys.view(W * S, K), nlp, gpe)
    splits, scat, sps, uc = routing.meta_from_virtual_route(vce, W, S, gpe, W // L, L)
    new_pl, rounds = swap.decide_swaps(load_g, pl, L, nlp, C)
    nmoves = 0
    if new_pl is not None:
        nmoves = sum(len(m) for m in swap.net_moves(pl.p2l, new_pl.p2l, L, nlp))
    chunks = sps.long().view(W, W, gpe).sum(2)
    return {
        f"{name}.dims": np.array([W, L, G, K, S, nlp, zipf_s * 10, seed], dtype=np.int64),
        f"{name}.topk": npi(topk, np.int16),
        f"{name}.p2l": npi(pl.p2l),
        f"{name}.phys": npi(phys, np.int16),
        f"{name}.splits": npi(splits),
        f"{name}.m_r": npi(chunks.sum(0), np.int64),
        f"{name}.uc": npi(uc),
        f"{name}.scatter_sum": np.array([int((scat.long() * torch.arange(1, scat.numel() + 1).view_as(scat)).sum())],
                                        dtype=np.int64),
        f"{name}.caps": np.array([caps.recv_cap, caps.dispatch_recv, caps.dispatch_stage, caps.dispatch_relay,
                                  caps.combine_send, caps.combine_conv, caps.combine_wire, caps.pair_cap],
                                 dtype=np.int64),
        f"{name}.swap": np.array([rounds, nmoves], dtype=np.int64),
        f"{name}.p2l_swapped": npi(new_pl.p2l) if new_pl is not None else npi(pl.p2l),
    }


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <checkout of the reference project>" % sys.argv[0])
    root = sys.argv[1]
    mods = load_reference(root)
    gen = torch.Generator().manual_seed(1)
    cases = {}
    topo = [(1, 1, 16, 4, 8), (2, 2, 16, 4, 16), (4, 4, 32, 8, 24), (8, 8, 32, 8, 16), (8, 4, 32, 8, 24),
            (8, 2, 32, 8, 16), (4, 2, 32, 8, 24), (2, 1, 16, 4, 16), (16, 4, 128, 8, 16), (8, 4, 128, 8, 40)]
    n = 0
    for (R, L, G, K, S) in topo:
        for shift in (0, 1):
            for C in (0.25, 0.0, 0.5):
                if C != 0.25 and (shift or R > 8):
                    continue
                c = route_case(mods, R, L, G, K, S, G // R + 2, C, gen, shift)
                for k, v in c.items():
                    cases[f"c{n}.{k}"] = v
                n += 1
    cases["n_cases"] = np.array([n], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "planner_cases.npz"), **cases)
    print("planner cases:", n)

    sw = {}
    m = 0
    for (R, L, G) in [(4, 4, 32), (8, 4, 32), (8, 8, 128), (16, 4, 128), (4, 2, 32), (8, 8, 384)]:
        for _ in range(2):
            rec = swap_sequence(mods, R, L, G, 6, gen)
            for k, v in rec.items():
                sw[f"s{m}.{k}"] = v
            m += 1
    sw["n_seq"] = np.array([m], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "swap_cases.npz"), **sw)
    print("swap sequences:", m)

    cfg = {}
    cfg.update(config_case(mods, "qwen30b_w8", 8, 8, 128, 8, 512, 0, 0.25, False))
    cfg.update(config_case(mods, "qwen235b_w2", 2, 2, 128, 8, 512, 1.0, 0.25, True))
    cfg.update(config_case(mods, "qwen235b_w4", 4, 4, 128, 8, 512, 1.0, 0.25, True))
    cfg.update(config_case(mods, "qwen235b_w8", 8, 8, 128, 8, 512, 1.0, 0.25, True))
    cfg.update(config_case(mods, "k2_w8", 8, 8, 384, 8, 512, 1.2, 0.25, True))
    cfg.update(config_case(mods, "qwen235b_w8_l4", 8, 4, 128, 8, 512, 1.0, 0.25, True))
    cfg.update(config_case(mods, "qwen235b_w8_l2", 8, 2, 128, 8, 512, 1.0, 0.25, True))
    np.savez_compressed(os.path.join(HERE, "config_cases.npz"), **cfg)
    for k in sorted(cfg):
        if k.endswith(".m_r") or k.endswith(".caps") or k.endswith(".swap"):
            print(k, cfg[k].tolist())


if __name__ == "__main__":
    main()
