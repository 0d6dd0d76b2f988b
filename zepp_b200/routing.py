"""Routing helpers on the host side: the slack as an exact rational, the capacity record and the
init-time capacity sizing.  The router itself runs on the device (csrc/planner.cuh); sizing calls
it as every rank in turn on this rank's GPU, which is how one process derives the same provable
capacities the reference computes with its host router (python/zepp/routing.py:400-458)."""
import math
from dataclasses import dataclass

import numpy as np
import torch

from . import constants
from ._ext import C


def c_rational(Cf: float):
    """Routing slack C as an exact fraction (num, den) in lowest terms with den a power of two (at most 2**16);
    a C that is not such a dyadic rational is an assertion error, as in the reference (python/zepp/routing.py:26-33)."""
    from fractions import Fraction
    if not (math.isfinite(Cf) and Cf >= 0):
        raise AssertionError(f"router_c must be finite and >= 0: {Cf}")
    scaled = round(Cf * 65536)
    if abs(scaled / 65536 - Cf) >= 1e-12:
        raise AssertionError(f"router_c {Cf} is not a dyadic rational")
    frac = Fraction(scaled, 65536)
    return frac.numerator, frac.denominator


@dataclass
class Capacities:
    recv_cap: int          # rows a rank may receive / compute
    dispatch_recv: int
    dispatch_stage: int
    dispatch_relay: int
    combine_send: int
    combine_conv: int
    combine_wire: int
    pair_cap: int          # rows on one (source, destination) pair

    def as_list(self):
        return [self.recv_cap, self.dispatch_recv, self.dispatch_stage, self.dispatch_relay, self.combine_send,
                self.combine_conv, self.combine_wire, self.pair_cap]


def virtual_route(phys, nlp, gpe):
    """Physical slots -> virtual GEMM group ids (the pad group is local index 0)."""
    p = phys.long()
    return ((p // nlp) * gpe + 1 + p % nlp).int()


def device_route_all(topk_all, placement, nlp, L, c_num, c_den, device):
    """Route every rank's entries on `device` -> (phys [R, S, K] int32 cuda, tables dict of numpy arrays)."""
    R, S, K = topk_all.shape
    G = placement.num_experts
    topk = topk_all.to(device=device, dtype=torch.int32).contiguous()
    loads = torch.stack([torch.bincount(topk[r].reshape(-1).long(), minlength=G) for r in range(R)]).int().contiguous()
    l2p = placement.l2p.to(device=device, dtype=torch.int32).contiguous()
    lcnts = placement.lcnts.to(device=device, dtype=torch.int32).contiguous()
    off = C.route_ws_offsets(G, R)
    CM = min(R, 32)
    ws = torch.zeros(C.route_workspace_ints(G, R), dtype=torch.int32, device=device)
    extra = np.zeros((G, R, CM), dtype=np.int64)
    phys = torch.empty(R, S, K, dtype=torch.int32, device=device)
    for i in range(R):
        C.route_tables_only(loads, l2p, lcnts, i, nlp, L, c_num, c_den, ws)     # budgets before the vacate pass
        extra[:, i, :] = ws[off["extra"]:off["extra"] + G * CM].view(G, CM).cpu().numpy()
        phys[i], _ = C.route_fused(topk[i], loads, l2p, lcnts, i, nlp, L, c_num, c_den, ws)
    w = ws.cpu().numpy().astype(np.int64)
    tab = dict(rep=w[off["rep"]:off["rep"] + G * CM].reshape(G, CM), c=w[off["c"]:off["c"] + G],
               U=w[off["U"]:off["U"] + G], M=w[off["M"]:off["M"] + G * R * CM].reshape(G, R, CM), extra=extra)
    return phys, tab


def compute_capacities(topk_all, placements, nlp, L, Cf, group=None, device=None) -> Capacities:
    """Provable buffer capacities from the routes of every placement the layer may run on."""
    device = device or torch.device("cuda")
    R, S, K = topk_all.shape
    W, NN, gpe = R, R // L, nlp + 1
    c_num, c_den = c_rational(Cf)
    cush = constants.CAPACITY_CUSHION_PER_RANK
    recv_ub = pair_ub = ext_dst_max = 0
    ext_pair = np.zeros((W, W), dtype=np.int64)
    dmax = np.zeros(7, dtype=np.int64)
    for pl in placements:
        phys, tab = device_route_all(topk_all, pl, nlp, L, c_num, c_den, device)
        rep, cnt, U, M, extra = tab["rep"], tab["c"], tab["U"], tab["M"], tab["extra"]
        hosted = (np.arange(rep.shape[1])[None, :] < cnt[:, None]) & (rep >= 0)
        gi, ji = np.nonzero(hosted)
        dst = rep[gi, ji]
        r_ub = np.bincount(dst, weights=U[gi], minlength=W).astype(np.int64)
        p_ub = np.zeros((W, W), dtype=np.int64)
        e_pair = np.zeros((W, W), dtype=np.int64)
        for i in range(W):
            p_ub[i] = np.bincount(dst, weights=(M[gi, i, ji] + extra[gi, i, ji]), minlength=W)
            e_pair[i] = np.bincount(dst, weights=extra[gi, i, ji], minlength=W)
        recv_ub = max(recv_ub, int(r_ub.max()))
        pair_ub = max(pair_ub, int(p_ub.max()))
        ext_dst_max = max(ext_dst_max, int(e_pair.sum(0).max()))
        ext_pair = np.maximum(ext_pair, e_pair)
        meta = C.routed_meta_full(R, L, S, K, nlp, gpe, vce=virtual_route(phys.view(R * S, K), nlp, gpe).contiguous())
        dmax = np.maximum(dmax, meta["demands"][:7].cpu().numpy())
    cushion = ext_dst_max + cush * W
    recv_cap = recv_ub + cush * W
    Em = ext_pair.reshape(NN, L, NN, L).sum(3).sum(1)
    np.fill_diagonal(Em, 0)
    cushion_relay = constants.RELAY_SLOTS * ((int(Em.max()) + L - 1) // L + 1) + cush * W
    vals = torch.tensor([recv_cap, max(int(dmax[1]) + cushion, recv_cap), int(dmax[2]) + cushion,
                         int(dmax[3]) + cushion_relay, max(int(dmax[0]) + cushion, recv_cap), int(dmax[4]) + cushion,
                         int(dmax[5]) + cushion, pair_ub + cushion], dtype=torch.int64)
    if group is not None and torch.distributed.is_available() and torch.distributed.is_initialized() \
            and hasattr(group, "size") and not getattr(group, "is_local", False) and group.size() > 1:
        v = vals.to(device)
        torch.distributed.all_reduce(v, op=torch.distributed.ReduceOp.MAX, group=group)
        vals = v.cpu()
    return Capacities(*[int(x) for x in vals])
