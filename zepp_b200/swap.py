"""Host-side helpers of the expert swap: reading the device decision's result block
(csrc/swap.cuh; layout of the reference's src/planner/swap_decide.cu) and the setup-time swap
orbit used for capacity sizing (python/zepp/swap.py:204-220)."""
import numpy as np
import torch

from . import constants
from ._ext import C
from .placement import Placement, rebuild_l2p


def parse_swap_block(blk, R, nlp, G, cap=constants.SWAP_MAX_MOVES):
    """int64 result block -> dict(rounds, total, err, moves[r] = [(dst slot, src rank, src slot, expert)],
    p2l int32 [R*nlp], load_g int64 [G])."""
    b = np.asarray(blk.cpu().numpy() if hasattr(blk, "cpu") else blk, dtype=np.int64)
    mv = b[3 + R:3 + R + 4 * R * cap].reshape(R, cap, 4)
    o = 3 + R + 4 * R * cap
    moves = [[tuple(int(v) for v in mv[r, i]) for i in range(int(b[3 + r]))] for r in range(R)]
    return dict(rounds=int(b[0]), total=int(b[1]), err=int(b[2]), moves=moves,
                p2l=b[o:o + R * nlp].astype(np.int32), load_g=b[o + R * nlp:o + R * nlp + G])


def decide_swaps(load_g, placement: Placement, L, nlp, Cf, cap=constants.SWAP_MAX_MOVES, max_rounds=32,
                 device=None):
    """Device swap decision for a global load vector -> (new Placement or None, rounds, moves)."""
    device = device or torch.device("cuda")
    G = placement.num_experts
    R = placement.p2l.numel() // nlp
    loads = torch.zeros(R, G, dtype=torch.int32, device=device)
    loads[0] = torch.as_tensor(load_g).to(device=device, dtype=torch.int32)
    p2l = placement.p2l.to(device=device, dtype=torch.int32).clone()
    l2p = placement.l2p.to(device=device, dtype=torch.int32).clone()
    lcnts = placement.lcnts.to(device=device, dtype=torch.int32)
    out = torch.zeros(C.swap_decide_out_ints(R, G, nlp, cap), dtype=torch.int64, device=device)
    C.swap_decide(loads, p2l, l2p, lcnts, L, nlp, float(Cf), cap, max_rounds, out)
    res = parse_swap_block(out, R, nlp, G, cap)
    if res["rounds"] == 0:
        return None, 0, res["moves"]
    p2l_h = torch.from_numpy(res["p2l"].copy())
    return Placement(p2l_h, rebuild_l2p(p2l_h, G, R), placement.lcnts, placement.stats), res["rounds"], res["moves"]


def swap_orbit(load_g, placement: Placement, L, nlp, Cf, max_rounds=8, device=None):
    """Successive placements of the one-round-per-step swap sequence on a fixed demand."""
    out, cur = [], placement
    seen = {cur.p2l.numpy().tobytes()}
    for _ in range(max_rounds):
        nxt, _rounds, _ = decide_swaps(load_g, cur, L, nlp, Cf, max_rounds=1, device=device)
        if nxt is None:
            break
        key = nxt.p2l.numpy().tobytes()
        if key in seen:
            break
        seen.add(key)
        out.append(nxt)
        cur = nxt
    return out
