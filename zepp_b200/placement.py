"""Load-aware replicated expert placement (host, init-time).

A pure integer function of the per-node demand histogram, identical on every rank without
communication; semantics follow the reference's python/zepp/placement.py:41-225 bit for bit:
replicate the expert with the largest per-instance share (at most one instance per node), place
instances on nodes by (affinity, node load, node id), backfill leftover slots, snake the node's
instances over its ranks, ascending expert ids inside a rank.
"""
import heapq
from dataclasses import dataclass

import numpy as np
import torch

from .constants import SHARE_BITS


@dataclass
class Placement:
    p2l: torch.Tensor      # int32 [R * slots_per_rank]: expert of each physical slot, -1 empty
    l2p: torch.Tensor      # int32 [G, R]: physical slots hosting each expert, ascending, -1 pad
    lcnts: torch.Tensor    # int32 [G]: replica count
    stats: dict

    @property
    def num_experts(self) -> int:
        return int(self.lcnts.numel())

    def clone(self) -> "Placement":
        return Placement(self.p2l.clone(), self.l2p.clone(), self.lcnts.clone(), dict(self.stats))


def demand_histogram(topk_all: torch.Tensor, ranks_per_node: int, num_experts: int) -> torch.Tensor:
    """Routing [R, S, K] -> per-node expert demand [NN, G] (int64, on the routing's device)."""
    R = topk_all.shape[0]
    NN = R // ranks_per_node
    ids = topk_all.reshape(NN, -1).long()
    node = torch.arange(NN, device=ids.device).unsqueeze(1) * num_experts
    return torch.bincount((ids + node).reshape(-1), minlength=NN * num_experts).view(NN, num_experts)


def _replica_counts(load, nodes, total_slots):
    """Instances per expert: one each, then the spare slots go one at a time to the expert whose per-instance share
    (load << SHARE_BITS) // instances is largest (ties: lower id), never more than one instance per node."""
    G = len(load)
    if total_slots < G:
        raise AssertionError("fewer slots than experts")
    most = min(nodes, total_slots)
    counts = [1] * G
    if most <= 1:
        return counts
    # max-heap on the current share; an entry is pushed again only while its expert may still grow
    queue = [(-(int(v) << SHARE_BITS), g) for g, v in enumerate(load)]
    heapq.heapify(queue)
    for _ in range(total_slots - G):
        if not queue:
            break
        _, g = heapq.heappop(queue)
        counts[g] += 1
        if counts[g] < most:
            heapq.heappush(queue, (-((int(load[g]) << SHARE_BITS) // counts[g]), g))
    return counts


def rebuild_l2p(p2l: torch.Tensor, num_experts: int, ranks: int) -> torch.Tensor:
    """l2p [G, R] from p2l: every expert's physical slots in ascending order, -1 behind them."""
    table = [[] for _ in range(num_experts)]
    for slot, expert in enumerate(p2l.cpu().tolist()):       # ascending slots, so each list comes out sorted
        if expert >= 0:
            table[expert].append(slot)
    l2p = torch.full((num_experts, ranks), -1, dtype=torch.int32)
    for expert, slots in enumerate(table):
        if slots:
            l2p[expert, :len(slots)] = torch.tensor(slots, dtype=torch.int32)
    return l2p


def solve_placement(hist: torch.Tensor, ranks_per_node: int, slots_per_rank: int) -> Placement:
    h = hist.cpu().numpy().astype(np.int64)
    NN, G = h.shape
    L, nlp = ranks_per_node, slots_per_rank
    R = NN * L
    load = [int(v) for v in h.sum(0)]
    c = _replica_counts(load, NN, R * nlp)
    share = [(load[g] << SHARE_BITS) // c[g] for g in range(G)]
    free = [L * nlp] * NN
    node_load = [0] * NN
    hosts = np.zeros((G, NN), dtype=bool)
    spilled = 0
    for g in sorted(range(G), key=lambda g: (-share[g], g)):
        mine = []
        for inst in range(c[g]):
            cands = [u for u in range(NN) if free[u] > 0 and u not in mine]
            if not cands:
                spilled += c[g] - inst
                break
            u = min(cands, key=lambda u: (-int(h[u, g]), node_load[u], u))
            mine.append(u)
            free[u] -= 1
            node_load[u] += share[g]
        assert mine, "expert with no instance"
        hosts[g, mine] = True
    capped = [min(s, 1 << 32) for s in share]
    for u in range(NN):
        if free[u] > 0:
            spare = sorted((g for g in range(G) if not hosts[g, u]), key=lambda g: (-capped[g], g))
            hosts[spare[:free[u]], u] = True
    c_real = hosts.sum(1)
    share_real = [(load[g] << SHARE_BITS) // max(int(c_real[g]), 1) for g in range(G)]
    per_rank = [[] for _ in range(R)]
    for u in range(NN):
        inst = sorted(np.nonzero(hosts[:, u])[0].tolist(), key=lambda g: (-share_real[g], g))
        for pos, g in enumerate(inst):
            lane = pos % L if (pos // L) % 2 == 0 else L - 1 - pos % L
            per_rank[u * L + lane].append(g)
    p2l = np.full(R * nlp, -1, dtype=np.int32)
    for r, experts in enumerate(per_rank):
        assert len(experts) <= nlp, "rank over its slot count"
        p2l[r * nlp:r * nlp + len(experts)] = sorted(experts)
    p2l_t = torch.from_numpy(p2l)
    lcnts = torch.from_numpy(np.bincount(p2l[p2l >= 0], minlength=G).astype(np.int32))
    stats = {"replicas": int(c_real.sum()) - G, "spilled": spilled, "c_max": int(c_real.max()),
             "remote_rows_predicted": int((h * (~hosts).T).sum())}
    return Placement(p2l_t, rebuild_l2p(p2l_t, G, R), lcnts, stats)
