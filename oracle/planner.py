"""CPU oracle of the MoE-layer planner (TEST INFRASTRUCTURE, not product code).

A clean restatement, in plain Python/numpy loops, of the integer planning algorithms of the
reference (andronius-yang/zepp).  Only tests/, __graft_entry__.smoke() and bench.py's CPU
baseline may import this module; the product package never does.

Each function cites the reference lines whose *behaviour* it restates.  The restatement is
pinned in this repository by tests/golden/*.npz, which were produced by importing the
reference's own Python planner (tests/golden/make_golden.py) -- parity is pinned.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

SHARE_BITS = 20                 # python/zepp/placement.py:23
CUSHION_PER_RANK = 8            # python/zepp/constants.py:21
RELAY_SLOTS = 2                 # python/zepp/constants.py:22
SWAP_MAX_MOVES = 8              # python/zepp/constants.py:11


# --------------------------------------------------------------------------------------
# slack as an exact rational                                   python/zepp/routing.py:26-33
# --------------------------------------------------------------------------------------
def c_rational(C: float):
    assert math.isfinite(C) and C >= 0
    den = 1 << 16
    num = int(round(C * den))
    assert abs(num / den - C) < 1e-12, "router_c must be a dyadic rational"
    g = math.gcd(num, den) if num else den
    return num // g, den // g


# --------------------------------------------------------------------------------------
# placement                                                   python/zepp/placement.py:41-225
# --------------------------------------------------------------------------------------
@dataclass
class Placement:
    p2l: np.ndarray            # int32 [R*nlp] expert of each physical slot, -1 empty
    l2p: np.ndarray            # int32 [G, R] ascending physical slots per expert, -1 pad
    lcnts: np.ndarray          # int32 [G] replica count
    stats: dict = field(default_factory=dict)


def demand_histogram(topk_all: np.ndarray, L: int, G: int) -> np.ndarray:
    """[R, S, K] expert ids -> per-node demand [NN, G] (placement.py:41-51)."""
    R = topk_all.shape[0]
    NN = R // L
    hist = np.zeros((NN, G), dtype=np.int64)
    for r in range(R):
        hist[r // L] += np.bincount(topk_all[r].reshape(-1).astype(np.int64), minlength=G)
    return hist


def replica_counts(load, nodes: int, total_slots: int):
    """Greedy replication of the expert with the largest per-instance share, at most one
    instance per node (placement.py:77-95).  Max-heap by (share, lower id first)."""
    import heapq
    G = len(load)
    assert total_slots >= G
    c = [1] * G
    cap = min(nodes, total_slots)
    heap = [(-(int(load[g]) << SHARE_BITS), g) for g in range(G)]
    heapq.heapify(heap)
    spare = total_slots - G
    while spare > 0 and heap:
        _, g = heapq.heappop(heap)
        if c[g] >= cap:
            continue
        c[g] += 1
        spare -= 1
        if c[g] < cap:
            heapq.heappush(heap, (-((int(load[g]) << SHARE_BITS) // c[g]), g))
    return c


def solve_placement(hist: np.ndarray, L: int, nlp: int) -> Placement:
    """hist [NN, G] -> tables (placement.py:98-212): node choice by (affinity desc, node
    load asc, node id asc); backfill of leftover slots by share; snake over the node's
    ranks; ascending expert ids inside a rank."""
    hist = np.asarray(hist, dtype=np.int64)
    NN, G = hist.shape
    R = NN * L
    load = hist.sum(0)
    c = replica_counts(load, NN, R * nlp)
    share = [(int(load[g]) << SHARE_BITS) // c[g] for g in range(G)]
    order = sorted(range(G), key=lambda g: (-share[g], g))
    free = [L * nlp] * NN
    node_load = [0] * NN
    on = np.zeros((G, NN), dtype=bool)
    spilled = 0
    for g in order:
        hosted = []
        for inst in range(c[g]):
            best = -1
            for u in range(NN):
                if free[u] <= 0 or u in hosted:
                    continue
                if best < 0:
                    best = u
                    continue
                a, b = int(hist[u, g]), int(hist[best, g])
                if a > b or (a == b and node_load[u] < node_load[best]):
                    best = u
            if best < 0:
                spilled += c[g] - inst
                break
            hosted.append(best)
            free[best] -= 1
            node_load[best] += share[g]
        assert hosted, "expert with no instance"
        for u in hosted:
            on[g, u] = True
    if sum(free) > 0:
        share_c = [min(s, 1 << 32) for s in share]
        for u in range(NN):
            if free[u] <= 0:
                continue
            cand = sorted((g for g in range(G) if not on[g, u]), key=lambda g: (-share_c[g], g))
            for g in cand[:free[u]]:
                on[g, u] = True
    c_real = on.sum(1)
    share2 = [(int(load[g]) << SHARE_BITS) // max(int(c_real[g]), 1) for g in range(G)]
    pairs = []                                   # (expert, rank)
    for u in range(NN):
        inst = sorted((g for g in range(G) if on[g, u]), key=lambda g: (-share2[g], g))
        for pos, g in enumerate(inst):
            lane = pos % L
            if (pos // L) % 2 == 1:
                lane = L - 1 - lane
            pairs.append((g, u * L + lane))
    p2l = np.full(R * nlp, -1, dtype=np.int32)
    per_rank = [[] for _ in range(R)]
    for g, r in pairs:
        per_rank[r].append(g)
    for r in range(R):
        per_rank[r].sort()
        assert len(per_rank[r]) <= nlp, "rank over its slot count"
        for j, g in enumerate(per_rank[r]):
            p2l[r * nlp + j] = g
    l2p = rebuild_l2p(p2l, G, R)
    lcnts = np.bincount(p2l[p2l >= 0], minlength=G).astype(np.int32)
    remote = int((hist * (~on).T).sum())
    return Placement(p2l, l2p, lcnts, dict(replicas=int(c_real.sum()) - G, spilled=spilled,
                                           c_max=int(c_real.max()), remote_rows_predicted=remote))


def rebuild_l2p(p2l, G: int, R: int) -> np.ndarray:
    """l2p from p2l: physical slots of each expert in ascending order (placement.py:215-225)."""
    l2p = np.full((G, R), -1, dtype=np.int32)
    fill = [0] * G
    for phys, e in enumerate(np.asarray(p2l).tolist()):
        if e >= 0:
            l2p[e, fill[e]] = phys
            fill[e] += 1
    return l2p


# --------------------------------------------------------------------------------------
# route tables                                                  python/zepp/routing.py:40-133
# --------------------------------------------------------------------------------------
def instance_phys_of_rank(l2p, lcnts, nlp: int, R: int) -> np.ndarray:
    G = l2p.shape[0]
    ipr = np.full((G, R), -1, dtype=np.int64)
    for g in range(G):
        for j in range(min(int(lcnts[g]), l2p.shape[1])):
            p = int(l2p[g, j])
            if p >= 0:
                ipr[g, p // nlp] = p
    return ipr


def rotation_round(i: int, j: int, L: int, NN: int) -> int:
    return (((j // L) - (i // L)) % NN) * L + (((j % L) - (i % L)) % L)


def route_bounds(D: int, c: int, c_num: int, c_den: int):
    """(U, Lb) of one expert (routing.py:71-77)."""
    if c <= 0:
        return 0, 0
    U = -((-(c_den + c_num) * D) // (c_den * c))
    Lb = ((c_den - c_num) * D) // (c_den * c)
    return U, Lb


def route_tables(d: np.ndarray, ipr: np.ndarray, L: int, c_num: int, c_den: int):
    """Rotation water-fill (routing.py:80-119).  d [R, G] demand of source i for expert g.
    Returns dict(M [G,R,Cmax], rep [G,Cmax], c [G], D, U, Lb [G], fill [G,Cmax], Cmax)."""
    d = np.asarray(d, dtype=np.int64)
    R, G = d.shape
    NN = R // L
    reps = [[r for r in range(R) if ipr[g, r] >= 0] for g in range(G)]
    Cmax = max(1, max(len(x) for x in reps))
    rep = np.full((G, Cmax), -1, dtype=np.int64)
    c = np.zeros(G, dtype=np.int64)
    M = np.zeros((G, R, Cmax), dtype=np.int64)
    fill = np.zeros((G, Cmax), dtype=np.int64)
    Dv = d.sum(0)
    Uv = np.zeros(G, dtype=np.int64)
    Lv = np.zeros(G, dtype=np.int64)
    for g in range(G):
        cg = len(reps[g])
        c[g] = cg
        rep[g, :cg] = reps[g]
        D = int(Dv[g])
        assert D == 0 or cg >= 1, "demand for an expert with no replica"
        U, Lb = route_bounds(D, cg, c_num, c_den)
        Uv[g], Lv[g] = U, Lb
        left = [int(d[i, g]) for i in range(R)]
        f = [0] * cg
        unassigned = D
        for p in range(R):
            du, dl = p // L, p % L
            for jj in range(cg):
                j = reps[g][jj]
                i = (((j // L) - du) % NN) * L + (((j % L) - dl) % L)
                deficit_others = sum(max(0, Lb - f[k]) for k in range(cg) if k != jj)
                take = min(left[i], U - f[jj], unassigned - deficit_others)
                take = max(take, 0)
                M[g, i, jj] = take
                f[jj] += take
                left[i] -= take
                unassigned -= take
        assert unassigned == 0 and all(v == 0 for v in left), "stranded demand"
        fill[g, :cg] = f
    return dict(M=M, rep=rep, c=c, D=Dv, U=Uv, Lb=Lv, fill=fill, Cmax=Cmax)


def water_fill_assign(topk_all: np.ndarray, ipr: np.ndarray, tab: dict, L: int) -> np.ndarray:
    """Deterministic ordinal assignment (routing.py:146-186): the o-th entry of (source i,
    expert g) in flat (token, k) order lands in the visit-ordered segment containing o."""
    R, S, K = topk_all.shape
    NN = R // L
    M, rep, c = tab["M"], tab["rep"], tab["c"]
    phys = np.empty((R, S, K), dtype=np.int64)
    for i in range(R):
        seen = {}
        visit = {}
        flat = topk_all[i].reshape(-1)
        out = phys[i].reshape(-1)
        for n in range(S * K):
            g = int(flat[n])
            if g not in visit:
                cg = int(c[g])
                order = sorted(range(cg), key=lambda jj: (rotation_round(i, int(rep[g, jj]), L, NN), jj))
                cum, acc = [], 0
                for jj in order:
                    acc += int(M[g, i, jj])
                    cum.append(acc)
                visit[g] = (order, cum)
            order, cum = visit[g]
            o = seen.get(g, 0)
            seen[g] = o + 1
            seg = sum(1 for v in cum if v <= o)
            assert seg < len(order), "ordinal beyond the segment table"
            out[n] = ipr[g, rep[g, order[seg]]]
    return phys


def lr_split(total: int, weights):
    """Largest-remainder split (routing.py:189-199): ties to the lower index."""
    W = sum(weights)
    n = len(weights)
    if total <= 0 or W <= 0:
        return [0] * n
    base = [total * w // W for w in weights]
    frac = [(total * w) % W for w in weights]
    rem = total - sum(base)
    for k in sorted(range(n), key=lambda k: (-frac[k], k))[:rem]:
        base[k] += 1
    return base


def vacate_budgets(d: np.ndarray, tab: dict):
    """release / extra [G, R, Cmax] (routing.py:202-225).

    Single-rank quirk kept for bit parity: with R == 1 the reference's table pass consumes its
    demand tensor in place (`left = d.t().contiguous()` aliases d when R == 1, routing.py:94,115),
    so the demand weights seen by the extra split are all zero and every extra budget is 0."""
    d = np.asarray(d, dtype=np.int64)
    R, G = d.shape
    if R == 1:
        d = np.zeros_like(d)
    Cmax = tab["Cmax"]
    release = np.zeros((G, R, Cmax), dtype=np.int64)
    extra = np.zeros((G, R, Cmax), dtype=np.int64)
    for g in range(G):
        for jj in range(int(tab["c"][g])):
            f, U, Lb = int(tab["fill"][g, jj]), int(tab["U"][g]), int(tab["Lb"][g])
            if f > Lb:
                w = [int(tab["M"][g, i, jj]) for i in range(R)]
                sp = lr_split(f - Lb, w)
                for i in range(R):
                    release[g, i, jj] = min(sp[i], w[i])
            if U > f:
                sp = lr_split(U - f, [int(d[i, g]) for i in range(R)])
                for i in range(R):
                    extra[g, i, jj] = sp[i]
    return release, extra


def vacate(topk_all, phys0, ipr, tab, release, extra, nlp: int, L: int) -> np.ndarray:
    """Per-token vacate pass, sequential per source rank (routing.py:242-297)."""
    R, S, K = topk_all.shape
    rep, c = tab["rep"], tab["c"]
    phys = phys0.copy()
    for i in range(R):
        home = i // L
        rel = release[:, i, :].copy()
        ext = extra[:, i, :].copy()
        for s in range(S):
            node_of = [int(phys[i, s, k]) // nlp // L for k in range(K)]
            while True:
                groups = {}                                   # node -> entries, first-touch order
                for k in range(K):
                    if node_of[k] != home:
                        groups.setdefault(node_of[k], []).append(k)
                if not groups:
                    break
                moved = False
                for n in sorted(groups, key=lambda x: (len(groups[x]), x)):
                    targets = [home] + [m for m in groups if m != n]
                    plan = []
                    for k in groups[n]:
                        g = int(topk_all[i, s, k])
                        cg = int(c[g])
                        jo = next(jj for jj in range(cg) if ipr[g, rep[g, jj]] == phys[i, s, k])
                        if rel[g, jo] <= 0:
                            plan = None
                            break
                        jt = None
                        for m in targets:
                            for jj in range(cg):
                                if rep[g, jj] // L == m and ext[g, jj] > 0:
                                    jt = jj
                                    break
                            if jt is not None:
                                break
                        if jt is None:
                            plan = None
                            break
                        plan.append((k, g, jo, jt))
                    if plan is None:
                        continue
                    for k, g, jo, jt in plan:
                        rel[g, jo] -= 1
                        ext[g, jo] += 1
                        ext[g, jt] -= 1
                        rel[g, jt] += 1
                        phys[i, s, k] = ipr[g, rep[g, jt]]
                        node_of[k] = int(rep[g, jt]) // L
                    moved = True
                    break
                if not moved:
                    break
    return phys


def reference_route(topk_all, pl: Placement, nlp: int, L: int, C: float):
    """Water-fill + vacate for all ranks (routing.py:228-299).  -> (phys int32 [R,S,K], info)."""
    topk_all = np.asarray(topk_all, dtype=np.int64)
    R, S, K = topk_all.shape
    G = int(pl.lcnts.shape[0])
    c_num, c_den = c_rational(C)
    ipr = instance_phys_of_rank(pl.l2p, pl.lcnts, nlp, R)
    d = np.stack([np.bincount(topk_all[r].reshape(-1), minlength=G) for r in range(R)]).astype(np.int64)
    tab = route_tables(d, ipr, L, c_num, c_den)
    phys0 = water_fill_assign(topk_all, ipr, tab, L)
    release, extra = vacate_budgets(d, tab)
    phys = vacate(topk_all, phys0, ipr, tab, release, extra, nlp, L) if R // L > 1 else phys0
    assert np.array_equal(np.asarray(pl.p2l, dtype=np.int64)[phys], topk_all), "conservation violated"
    return phys.astype(np.int32), dict(tables=tab, release=release, extra=extra, d=d, ipr=ipr, phys0=phys0)


# --------------------------------------------------------------------------------------
# virtual ids + routed metadata                                python/zepp/routing.py:306-331
# --------------------------------------------------------------------------------------
def virtual_route(phys, nlp: int, gpe: int) -> np.ndarray:
    p = np.asarray(phys, dtype=np.int64)
    return ((p // nlp) * gpe + 1 + p % nlp).astype(np.int32)


def routed_meta(vce: np.ndarray, R: int, S: int, gpe: int, NN: int, L: int):
    """(splits [E_virt], scatter_index [R*S,K], sps [R,E_virt], uc [R, R+NN]).

    A negative entry is a pad copy: it is counted nowhere and gets scatter_index -1.  The reference planner
    never sees such entries (its serving path routes pad rows to local experts, python/zepp/serving.py:106-160);
    for real copies the result equals the reference's on the routing with the pad rows removed."""
    vce = np.asarray(vce, dtype=np.int64)
    ntok, K = vce.shape
    E_virt = R * gpe
    flat = vce.reshape(-1)
    splits = np.bincount(flat[flat >= 0], minlength=E_virt).astype(np.int32)
    base = np.concatenate([[0], np.cumsum(splits)[:-1]]).astype(np.int64)
    nxt = base.copy()
    scatter = np.full(flat.shape[0], -1, dtype=np.int32)
    for n, e in enumerate(flat.tolist()):                    # stable rank in expert-sorted order
        if e < 0:
            continue
        scatter[n] = nxt[e]
        nxt[e] += 1
    sps = np.zeros((R, E_virt), dtype=np.int32)
    uc = np.zeros((R, R + NN), dtype=np.int32)
    for t in range(ntok):
        s = t // S
        owners = set()
        for e in vce[t].tolist():
            if e < 0:
                continue
            sps[s, e] += 1
            owners.add(e // gpe)
        for o in owners:
            uc[s, o] += 1
        for n in {o // L for o in owners}:
            uc[s, R + n] += 1
    return splits, scatter.reshape(ntok, K), sps, uc


# --------------------------------------------------------------------------------------
# demands                                                      python/zepp/capacity.py:30-55
# --------------------------------------------------------------------------------------
def demands_from_meta(sps, uc, W: int, L: int, gpe: int):
    """7 exact demands: recv_rows, dispatch_recv, dispatch_stage, dispatch_relay,
    combine_conv, combine_wire, pair_rows."""
    sps = np.asarray(sps, dtype=np.int64)
    uc = np.asarray(uc, dtype=np.int64)
    NN = W // L
    chunks = sps.reshape(W, W, gpe).sum(2)
    recv_rows = int(chunks.sum(0).max())
    pair = max(int(chunks.max()), 1)
    if NN == 1:
        return [max(recv_rows, 1), max(recv_rows, 1), 1, 1, 1, 1, pair]
    u, U = uc[:, :W], uc[:, W:]
    disp = recv_rows
    for dst in range(W):
        tot = 0
        for s in range(W):
            tot += int(u[s, dst]) if s // L == dst // L else int(U[s, dst // L])
        disp = max(disp, tot)
    T = np.zeros((NN, NN), dtype=np.int64)                   # union rows node ns -> node n
    for s in range(W):
        T[s // L] += U[s]
    stage = relay = conv = wire = 0
    for n in range(NN):
        for k in range(L):
            chunk = lambda ns: int(T[ns, n]) // L + (1 if k < int(T[ns, n]) % L else 0)  # noqa: E731
            stage = max(stage, sum(chunk(ns) for ns in range(NN) if ns != n))
            relay = max(relay, max(chunk(ns) for ns in range(NN) if ns != n))
            conv = max(conv, sum(int(chunks[tn * L + k, n * L:(n + 1) * L].sum()) for tn in range(NN) if tn != n))
            wire = max(wire, sum(int(U[tn * L + k, n]) for tn in range(NN) if tn != n))
    relay *= RELAY_SLOTS
    return [max(recv_rows, 1), max(disp, 1), max(stage, 1), max(relay, 1), max(conv, 1), max(wire, 1), pair]


# bit i of the violation mask <-> (demand index, capacity index); capacities are ordered as
# Capacities: recv_cap, dispatch_recv, dispatch_stage, dispatch_relay, combine_send,
# combine_conv, combine_wire, pair_cap        (capacity.py:59-62, tests/test_meta_device.py:43-48)
FIT_OVERLAP = ((0, 0), (1, 1), (2, 2), (3, 3), (0, 4), (4, 5), (5, 6))
FIT_DIRECT = ((0, 0), (6, 7))


def violation_mask(dem, caps, direct: bool) -> int:
    mask = 0
    if direct:
        if dem[0] > caps[0]:
            mask |= 1
        if dem[6] > caps[7]:
            mask |= 0x80
        return mask
    for bit, (di, ci) in enumerate(FIT_OVERLAP):
        if dem[di] > caps[ci]:
            mask |= 1 << bit
    return mask


# --------------------------------------------------------------------------------------
# capacities                                                   python/zepp/routing.py:400-458
# --------------------------------------------------------------------------------------
def compute_capacities(topk_all, placements, nlp: int, L: int, C: float):
    topk_all = np.asarray(topk_all, dtype=np.int64)
    R, S, K = topk_all.shape
    W, NN, gpe = R, R // L, nlp + 1
    recv_ub = pair_ub = ext_dst_max = 0
    ext_pair = np.zeros((W, W), dtype=np.int64)
    dmax = [0] * 7
    comb_send = 0
    for pl in placements:
        phys, info = reference_route(topk_all, pl, nlp, L, C)
        tab, extra = info["tables"], info["extra"]
        rep, c = tab["rep"], tab["c"]
        r_ub = np.zeros(W, dtype=np.int64)
        p_ub = np.zeros((W, W), dtype=np.int64)
        e_dst = np.zeros(W, dtype=np.int64)
        e_pair = np.zeros((W, W), dtype=np.int64)
        for g in range(rep.shape[0]):
            for jj in range(int(c[g])):
                j = int(rep[g, jj])
                r_ub[j] += int(tab["U"][g])
                for i in range(W):
                    p_ub[i, j] += int(tab["M"][g, i, jj]) + int(extra[g, i, jj])
                    e_pair[i, j] += int(extra[g, i, jj])
                    e_dst[j] += int(extra[g, i, jj])
        recv_ub = max(recv_ub, int(r_ub.max()))
        pair_ub = max(pair_ub, int(p_ub.max()))
        ext_dst_max = max(ext_dst_max, int(e_dst.max()))
        ext_pair = np.maximum(ext_pair, e_pair)
        vce = virtual_route(phys.reshape(R * S, K), nlp, gpe)
        _, _, sps, uc = routed_meta(vce, R, S, gpe, NN, L)
        dem = demands_from_meta(sps, uc, W, L, gpe)
        # dispatch "recv" of the sizing pass = the node-union receive regions (routing.py:339-365)
        dmax = [max(a, b) for a, b in zip(dmax, dem)]
        chunks = np.asarray(sps, dtype=np.int64).reshape(W, W, gpe).sum(2)
        comb_send = max(comb_send, max(int(chunks.sum(0).max()), 1))
    cushion = ext_dst_max + CUSHION_PER_RANK * W
    recv_cap = recv_ub + CUSHION_PER_RANK * W
    E = ext_pair.reshape(NN, L, NN, L).sum(3).sum(1)
    np.fill_diagonal(E, 0)
    cushion_relay = RELAY_SLOTS * ((int(E.max()) + L - 1) // L + 1) + CUSHION_PER_RANK * W
    return [recv_cap, max(dmax[1] + cushion, recv_cap), dmax[2] + cushion, dmax[3] + cushion_relay,
            max(comb_send + cushion, recv_cap), dmax[4] + cushion, dmax[5] + cushion, pair_ub + cushion]


# --------------------------------------------------------------------------------------
# plan blocks (single NVLink domain subset)         python/zepp/routing.py:462-623, 629-714
# --------------------------------------------------------------------------------------
DP_HEADER = 8


def dispatch_plan_words(L: int, NN: int) -> int:
    nseg = L + NN - 1
    return DP_HEADER + nseg + 1 + 3 * L + NN * (6 + 8 * L) + NN * (3 + L)


def dispatch_plan_head(sps, uc, W: int, L: int, gpe: int, rank: int, copies_per_rank: int, max_recv: int):
    """Header + send segments + round-0 triples of the dispatch plan block of `rank`
    (routing.py:510-554, 613-623).  The per-node relay tables that follow them in the
    reference's block are inter-node machinery and are left zero."""
    sps = np.asarray(sps, dtype=np.int64)
    uc = np.asarray(uc, dtype=np.int64)
    NN = W // L
    me_n, me_l = rank // L, rank % L
    u, U = uc[:, :W], uc[:, W:]
    chunks = sps.reshape(W, W, gpe).sum(2)
    P = [0] * dispatch_plan_words(L, NN)

    def region(s, dst):
        return int(U[s, dst // L]) if s // L != dst // L else int(u[s, dst])

    err = 0
    for s in range(W):
        for dst in range(W):
            cv, uv = int(chunks[s, dst]), int(u[s, dst])
            if not (0 <= uv <= cv and (uv > 0) == (cv > 0)):
                err |= 4
            if uv > int(U[s, dst // L]):
                err |= 8
        for n in range(NN):
            if int(U[s, n]) > int(u[s, n * L:(n + 1) * L].sum()):
                err |= 8
    seg = [0]
    for n in range(NN):
        if n == me_n:
            for dl in range(L):
                seg.append(seg[-1] + int(u[rank, n * L + dl]))
        else:
            seg.append(seg[-1] + int(U[rank, n]))
    nseg = L + NN - 1
    P[DP_HEADER:DP_HEADER + nseg + 1] = seg
    r0 = DP_HEADER + nseg + 1
    for dl in range(L):
        dst = me_n * L + dl
        P[r0 + 3 * dl:r0 + 3 * dl + 3] = [int(u[rank, dst]), seg[me_n + dl],
                                          sum(region(s, dst) for s in range(rank))]
    max_col = max(sum(region(s, dst) for s in range(W)) for dst in range(W))
    if max_col > max_recv:
        err |= 16
    if seg[nseg] > copies_per_rank:
        err |= 32
    P[0] = int(chunks[:, rank].sum())
    P[1] = seg[nseg]
    P[2] = int(u[rank, rank])
    P[3] = seg[me_n + me_l]
    P[4] = sum(region(s, rank) for s in range(rank))
    P[5] = err
    return P, r0 + 3 * L          # words, number of leading words that are defined here


def combine_tables(sps, W: int, gpe: int, rank: int):
    """send_off [W+1], send_rows [W], dst_off [W], lane_off [W+1] of `rank` on one node
    (routing.py:656-669 with same_node everywhere): C[s][d] = rows owner s returns to home d."""
    cnt = np.asarray(sps, dtype=np.int64).reshape(W, W, gpe).sum(2)      # [home, owner]
    C = cnt.T                                                            # [owner, home]
    rows_to = C[rank]
    send_off = np.concatenate([[0], np.cumsum(rows_to)])
    dst_off = C[:rank].sum(0)
    lane_off = np.concatenate([[0], np.cumsum(C[:, rank])])
    return send_off, rows_to.copy(), dst_off, lane_off


# --------------------------------------------------------------------------------------
# swap decision                                                   python/zepp/swap.py:36-201
# --------------------------------------------------------------------------------------
def _node_out(L_r, L: int, C: float):
    lr = np.asarray(L_r, dtype=np.int64).reshape(-1, L)
    return lr.max(1).astype(np.float64) * L > (1.0 + C) * lr.sum(1).astype(np.float64)


def _swap_round(cur, w_slot, L_r, G: int, L: int, nlp: int, C: float):
    """One round (swap.py:54-113, per_pair == 1): list of (slot_h, e_h, slot_l, e_l)."""
    R = len(cur) // nlp
    NN = R // L
    out = _node_out(L_r, L, C)
    swaps = []
    Kc = min(8, nlp)
    for n in range(NN):
        ranks = sorted(range(L), key=lambda l: (-int(L_r[n * L + l]) * L + l))
        P = L // 2
        heavy = [n * L + ranks[q] for q in range(P)]
        light = [n * L + ranks[L - 1 - q] for q in range(P)]
        for h, lo in zip(heavy, light):
            LH, LL = int(L_r[h]), int(L_r[lo])
            if not (LH - LL > 1 and out[n]):
                continue
            hs = list(range(h * nlp, (h + 1) * nlp))
            ls = list(range(lo * nlp, (lo + 1) * nlp))
            BIG = 1 << 60
            hk = sorted(hs, key=lambda s: ((-int(w_slot[s]), int(cur[s])) if cur[s] >= 0 else (BIG, BIG), s))[:Kc]
            lk = sorted(ls, key=lambda s: ((int(w_slot[s]), int(cur[s])) if cur[s] >= 0 else (BIG, BIG), s))[:Kc]
            e_h_all = {int(cur[s]) for s in hs}
            e_l_all = {int(cur[s]) for s in ls}
            best, best_key = None, None
            for a, sh in enumerate(hk):
                eh, wh = int(cur[sh]), int(w_slot[sh])
                for b, sl in enumerate(lk):
                    el, wl = int(cur[sl]), int(w_slot[sl])
                    if eh < 0 or el < 0 or eh in e_l_all or el in e_h_all or eh == el or not wh > wl:
                        continue
                    gain = max(LH, LL) - max(LH - wh + wl, LL - wl + wh)
                    if gain < 1:
                        continue
                    key = gain * (G * G + 1) - (eh * G + el)
                    if best_key is None or key > best_key:          # first maximum in (a, b) order
                        best_key, best = key, (sh, eh, sl, el)
            if best is not None:
                swaps.append(best)
    return swaps


def decide_swaps(load_g, pl: Placement, L: int, nlp: int, C: float, cap: int = SWAP_MAX_MOVES,
                 max_rounds: int = 32):
    """-> (new p2l or None, rounds)   (swap.py:131-180)."""
    a0 = np.asarray(pl.p2l, dtype=np.int64)
    R = a0.shape[0] // nlp
    lg = np.asarray(load_g, dtype=np.int64)
    G = lg.shape[0]
    lc = np.maximum(np.asarray(pl.lcnts, dtype=np.int64), 1)
    w_slot = np.array([int(lg[e]) // int(lc[e]) if e >= 0 else 0 for e in a0.tolist()], dtype=np.int64)
    L_r = w_slot.reshape(R, nlp).sum(1)
    if not _node_out(L_r, L, C).any():
        return None, 0
    cur = a0.copy()
    rounds = 0
    for _ in range(max_rounds):
        swaps = _swap_round(cur, w_slot, L_r, G, L, nlp, C)
        if not swaps:
            break
        nxt = cur.copy()
        for sh, eh, sl, el in swaps:
            nxt[sh], nxt[sl] = el, eh
        if int((nxt != a0).reshape(R, nlp).sum(1).max()) > cap:
            break
        cur = nxt
        rounds += 1
        for sh, _eh, sl, _el in swaps:
            for sx in (sh, sl):
                e = int(cur[sx])
                w_new = int(lg[e]) // int(lc[e]) if e >= 0 else 0
                L_r[sx // nlp] += w_new - w_slot[sx]
                w_slot[sx] = w_new
    if rounds == 0:
        return None, 0
    return cur.astype(np.int32), rounds


def net_moves(p2l0, p2l_f, L: int, nlp: int):
    """Per-rank pull lists [(dst slot, src rank, src slot, expert)] (swap.py:183-201)."""
    a0, af = np.asarray(p2l0).tolist(), np.asarray(p2l_f).tolist()
    R = len(a0) // nlp
    where = {}
    for phys, e in enumerate(a0):
        if e >= 0:
            r = phys // nlp
            where[(r // L, e)] = (r, phys % nlp)
    moves = [[] for _ in range(R)]
    for phys, e in enumerate(af):
        if e >= 0 and a0[phys] != e:
            r = phys // nlp
            sr, ss = where[(r // L, e)]
            moves[r].append((phys % nlp, sr, ss, e))
    for m in moves:
        m.sort()
    return moves


def swap_orbit(load_g, pl: Placement, L: int, nlp: int, C: float, max_rounds: int = 8):
    """Successive placements of the one-round-per-step swap sequence (swap.py:204-220)."""
    G = int(pl.lcnts.shape[0])
    R = pl.p2l.shape[0] // nlp
    out, cur = [], pl
    seen = {bytes(np.asarray(cur.p2l, dtype=np.int32).tobytes())}
    for _ in range(max_rounds):
        nxt, _r = decide_swaps(load_g, cur, L, nlp, C, max_rounds=1)
        if nxt is None:
            break
        key = bytes(nxt.tobytes())
        if key in seen:
            break
        seen.add(key)
        cur = Placement(nxt, rebuild_l2p(nxt, G, R), pl.lcnts, pl.stats)
        out.append(cur)
    return out


def swap_result_block(load_g, pl: Placement, L: int, nlp: int, C: float, cap: int = SWAP_MAX_MOVES):
    """The int64 result block of the device swap decision (src/planner/swap_decide.cu:81-346
    as pinned by tests/test_swap_decide.py:57-86): [rounds, total moves, err, count[R],
    moves[R, cap, 4], p2l[R*nlp], load_g[G]]."""
    a0 = np.asarray(pl.p2l, dtype=np.int64)
    R = a0.shape[0] // nlp
    G = int(np.asarray(load_g).shape[0])
    new, rounds = decide_swaps(load_g, pl, L, nlp, C, cap)
    blk = np.zeros(3 + R + 4 * R * cap + R * nlp + G, dtype=np.int64)
    p2l_f = a0 if new is None else new.astype(np.int64)
    moves = net_moves(a0, p2l_f, L, nlp) if new is not None else [[] for _ in range(R)]
    blk[0] = rounds
    blk[1] = sum(len(m) for m in moves)
    mv = blk[3 + R:3 + R + 4 * R * cap].reshape(R, cap, 4)
    for r in range(R):
        blk[3 + r] = len(moves[r])
        for i, m in enumerate(moves[r]):
            mv[r, i] = m
    o = 3 + R + 4 * R * cap
    blk[o:o + R * nlp] = p2l_f
    blk[o + R * nlp:] = np.asarray(load_g, dtype=np.int64)
    return blk


def lane_arm_expect(moves_r, nlp: int, epoch: int, stag_addr, sentinel: int = -7):
    """Expected swap-lane metadata of one rank (tests/test_lane_device.py:36-58): gate words of
    the unchanged slots (both matrices), schedule word per group (bit 30 = incoming slot, low bits
    = rank inside its class; the pad group counts as unchanged) and staging overrides."""
    gpe = nlp + 1
    gate = np.full(2 * gpe, sentinel, dtype=np.int64)
    sched = np.full(gpe, sentinel, dtype=np.int32)
    ovr = [np.full(gpe, sentinel, dtype=np.int64) for _ in (0, 1)]
    if not moves_r:
        return gate, sched, ovr
    changed = {m[0] for m in moves_r}
    for i, m in enumerate(moves_r):
        ovr[0][1 + m[0]] = stag_addr[0][i]
        ovr[1][1 + m[0]] = stag_addr[1][i]
    nf = nd = 0
    for s in range(gpe):
        if s >= 1 and (s - 1) in changed:
            sched[s] = (1 << 30) | nd
            nd += 1
        else:
            sched[s] = nf
            nf += 1
            if s >= 1:
                gate[s] = epoch
                gate[gpe + s] = epoch
    return gate, sched, ovr
