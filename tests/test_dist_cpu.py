"""Multi-process host logic on CPU (gloo, world_size 2): the bootstrap all-gather of the arena
handles and the per-rank sharding of a workload (no GPU, no kernels)."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from zepp_b200 import EPMoEConfig
    from zepp_b200 import workloads as wl
    from zepp_b200.placement import demand_histogram, solve_placement
    from zepp_b200.runtime import gather_blobs
    blob = bytes([rank]) * 64
    allb = gather_blobs(dist.group.WORLD, blob)
    ok = allb == b"".join(bytes([r]) * 64 for r in range(world))
    # every rank derives the same routing and placement from the seed, and hosts a disjoint slot range
    shape, S, ids, wts, _, _ = wl.make("qwen3-30b", world, S=64)
    cfg = EPMoEConfig(shape=shape, ranks=world, ranks_per_node=world, max_tokens_per_rank=S)
    pl = solve_placement(demand_histogram(ids, world, shape.num_experts), world, cfg.slots_per_rank)
    digest = torch.tensor([int(pl.p2l.long().sum()), int(ids.long().sum())])
    gathered = [torch.zeros_like(digest) for _ in range(world)]
    dist.all_gather(gathered, digest)
    ok &= all(torch.equal(g, digest) for g in gathered)
    nlp = cfg.slots_per_rank
    mine = {int(e) for e in pl.p2l[rank * nlp:(rank + 1) * nlp].tolist() if e >= 0}
    sizes = [None] * world
    dist.all_gather_object(sizes, sorted(mine))
    ok &= sum(len(s) for s in sizes) == shape.num_experts and len(set().union(*map(set, sizes))) == shape.num_experts
    q.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_bootstrap_and_sharding_world2():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True), (1, True)], res
