"""Run under torch.distributed.run with one process per GPU: builds the layer across real GPUs
(CUDA IPC arenas, peer loads / stores over NVLink), runs a few steps and checks every rank's
output against the CPU oracle.  Used by tests/test_multi_gpu.py; prints one line per rank."""
import argparse
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--strategy", default="overlap")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--ranks-per-node", type=int, default=0)
    ap.add_argument("--swap", type=int, default=0)
    ap.add_argument("--zipf", type=float, default=0.0, help="popularity exponent (default 1.0, 1.2 with swap)")
    ap.add_argument("--drift", type=float, default=0.0, help="fraction of expert ranks re-permuted before every later step")
    ap.add_argument("--prime-seed", type=int, default=0, help="prime on a drifted batch drawn with this seed (0: on batch 0)")
    a = ap.parse_args()
    from oracle import layer as ol
    from zepp_b200 import EPMoE, EPMoEConfig, ModelShape
    from zepp_b200 import workloads as wl

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    shape = ModelShape(32, 8, 512, 256, act="swiglu")
    S = a.tokens
    cfg = EPMoEConfig(shape=shape, ranks=world, ranks_per_node=a.ranks_per_node or world, max_tokens_per_rank=S,
                      comm_strategy=a.strategy, swap=bool(a.swap))
    gen = torch.Generator().manual_seed(5)
    p = wl.popularity(shape.num_experts, a.zipf or (1.2 if a.swap else 1.0), gen)
    ids, wts = wl.routing(world, S, shape.topk, p, gen)
    layer = EPMoE(cfg, dist.group.WORLD, ids, ids)
    W1 = torch.stack([wl.expert_w1(e, shape) for e in range(shape.num_experts)])
    W2 = torch.stack([wl.expert_w2(e, shape) for e in range(shape.num_experts)])
    layer.load_weights(lambda e: W1[e], lambda e: W2[e])
    import numpy as np
    from oracle import planner as op
    # persistent device tensors: every step() replays ONE captured graph while the routing in them changes
    ids_d, w_d = ids[rank].cuda().contiguous(), wts[rank].cuda().contiguous()
    x_d = torch.empty(S, shape.hidden, dtype=torch.bfloat16, device="cuda")
    ids_p, wts_p = ids, wts
    if a.prime_seed:          # a batch of another popularity: the priming pass itself decides moves
        gen_p = torch.Generator().manual_seed(a.prime_seed)
        ids_p, wts_p = wl.routing(world, S, shape.topk, wl.drift(p, a.drift or 0.5, gen_p), gen_p)
    layer.prime(ids_p[rank].cuda().contiguous(), wts_p[rank].cuda().contiguous())
    pl0 = layer.placement
    cur = op.Placement(pl0.p2l.numpy().copy(), pl0.l2p.numpy().copy(), pl0.lcnts.numpy())
    L = cfg.ranks_per_node

    def expect_swap(ids_step, cur):
        load_g = np.bincount(ids_step.numpy().reshape(-1), minlength=shape.num_experts)
        new, rounds = op.decide_swaps(load_g, cur, L, cfg.slots_per_rank, cfg.router_c)
        if not rounds:
            return cur, 0
        moves = op.net_moves(cur.p2l, new, L, cfg.slots_per_rank)
        return op.Placement(new, op.rebuild_l2p(new, shape.num_experts, world), cur.lcnts), sum(len(m) for m in moves)

    if a.swap:
        cur, n_prime = expect_swap(ids_p, cur)       # the priming pass decides too (and moves the weights)
        prime_ok = bool(np.array_equal(layer.tables("p2l")[0].cpu().numpy(), cur.p2l)) and layer.swap_moves == n_prime
    ok = True
    plan_ok = prime_ok if a.swap else True
    moved = n_prime if a.swap else 0
    worst = 0.0
    for step in range(a.steps):
        if step:
            if a.drift:
                p = wl.drift(p, a.drift, gen)
            ids, wts = wl.routing(world, S, shape.topk, p, gen)
            ids_d.copy_(ids[rank])
            w_d.copy_(wts[rank])
        x = wl.tokens(rank, S, shape.hidden, seed=step)
        x_d.copy_(x)
        if step == 0:
            plan = layer.prepare(ids_d, w_d)
            y = layer.forward(x_d, plan)
        else:
            y = layer.step(ids_d, w_d, x_d)
        layer.check()
        if a.swap:
            cur, n_moves = expect_swap(ids, cur)
            plan_ok &= bool(np.array_equal(layer.tables("p2l")[0].cpu().numpy(), cur.p2l)) and layer.swap_moves == n_moves
            moved += n_moves
        ref = ol.moe_reference_fp32(x, ids[rank], wts[rank], W1, W2)
        refb = ol.moe_reference_bf16_points(x, ids[rank], wts[rank], W1, W2).float()
        yc = y.float().cpu()
        err = float((yc - ref).abs().max())
        worst = max(worst, err)
        ok &= bool(torch.allclose(yc, ref, rtol=2e-2, atol=2e-2))
        scale = float(refb.abs().max())
        ok &= float((yc - refb).abs().max()) <= 1.5e-2 * scale and float((yc - refb).norm() / refb.norm()) <= 5e-3
    ok &= plan_ok
    moves = moved
    flag = torch.tensor([0 if ok else 1], device="cuda")
    dist.all_reduce(flag)
    print(f"[dist_layer_check] rank {rank}/{world} {a.strategy}: {'PASS' if ok else 'FAIL'} max|err| {worst:.4g} swap decisions {'ok' if plan_ok else 'DIFFER'} moves (prime + steps) {moves}", flush=True)
    layer.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 0 else 1)


if __name__ == "__main__":
    main()
