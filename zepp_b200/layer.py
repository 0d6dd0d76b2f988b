"""EPMoE: the expert-parallel MoE layer behind the reference's Python API
(python/zepp/layer.py:36-225):

    layer = EPMoE(cfg, group, sizing_routing=..., pool_routing=...)   # collective
    layer.load_weights(w1_of, w2_of)          # expert -> [ffn1, H] / [H, ffn]
    layer.prime(topk_ids, topk_weights)
    plan = layer.prepare(topk_ids, topk_weights)    # loads, (swap decision), route, metadata
    y = layer.forward(x, plan)                      # dispatch_gemm -> activation -> gemm_combine

Everything per step runs on the GPU through libzepp_b200.so: planning is integer CUDA kernels,
the two grouped GEMMs are tcgen05 kernels with the token transfers inside them (overlap) or beside
them (direct), and nothing is read back on the host inside a step.  Unlike the reference, whose
device planning needs two or more nodes (python/zepp/layer.py:66), device planning is always on.
"""
import torch

from . import constants
from .capacity import CapacityExceeded, Demands, violations
from .config import EPMoEConfig
from .placement import Placement, demand_histogram, solve_placement
from .planner import Plan
from .routing import c_rational, compute_capacities
from .runtime import LayerHandle, Runtime, make_cfg
from .swap import swap_orbit


def activation(h, shape, out=None):
    """The expert activation between the GEMMs as a torch op (the fused kernels apply the same
    function in their epilogue; python/zepp/layer.py:20-27)."""
    if shape.act == "gelu":
        return torch.nn.functional.gelu(h)
    ffn = shape.ffn_hidden
    return torch.mul(torch.nn.functional.silu(h[:, :ffn]), h[:, ffn:], out=out)


def token_buckets(cfg):
    """Token counts a layer captures a step for: k, 2k, 4k, ... and max_tokens_per_rank (all multiples of top-k),
    as the reference's serving path pads to (python/zepp/serving.py:42-50)."""
    k, top = cfg.shape.topk, cfg.max_tokens_per_rank
    out, s = [], k
    while s < top:
        out.append(s)
        s *= 2
    return out + [top]


class Marks:
    """Optional bracket marks for benchmarking (a callable per boundary)."""

    def __call__(self, name):
        pass


class LocalGroup:
    """Stand-in for a process group when all ranks live in this process (single-GPU emulation)."""
    is_local = True

    def __init__(self, rank, world):
        self._rank, self._world = rank, world

    def rank(self):
        return self._rank

    def size(self):
        return self._world


_ERR_NAMES = {1: "a device-side wait ran out", 2: "the step exceeded the buffer capacities",
              4: "an index table entry was out of range", 8: "the router could not place all rows"}


def plan_layer(cfg, sizing_routing, pool_routing, device, group):
    """Set-up planning shared by every way of building a layer: the placement from the pool routing's demand, and
    buffer capacities that hold the sizing batch on that placement and on every placement its swap orbit can reach
    (python/zepp/layer.py:53-62).  Collective over `group` when it is a process group (capacities are max-reduced)."""
    shape = cfg.shape
    demand = demand_histogram(pool_routing.to(device), cfg.ranks_per_node, shape.num_experts).cpu()
    placement = solve_placement(demand, cfg.ranks_per_node, cfg.slots_per_rank)
    sizing = sizing_routing.cpu()
    reachable = [placement]
    if cfg.swap:
        load = torch.bincount(sizing.reshape(-1).long(), minlength=shape.num_experts)
        reachable.extend(swap_orbit(load, placement, cfg.ranks_per_node, cfg.slots_per_rank, cfg.router_c, device=device))
    caps = compute_capacities(sizing, reachable, cfg.slots_per_rank, cfg.ranks_per_node, cfg.router_c, group, device=device)
    return placement, caps


class EPMoE(torch.nn.Module):
    def __init__(self, cfg: EPMoEConfig, group, sizing_routing, pool_routing, probs_own=None,
                 dtype=torch.bfloat16, _runtime=None):
        """sizing_routing [R, S, K]: expert ids of a representative batch (sizes the buffers from the
        provable routing bounds); pool_routing [R, S', K]: ids the placement is planned from;
        probs_own is accepted for signature compatibility (gate weights are set by prepare)."""
        super().__init__()
        assert dtype == torch.bfloat16, "the B200 kernels compute in bf16 with fp32 accumulation"
        self.cfg, self.group, self.dtype = cfg, group, dtype
        self.rank = group.rank()
        shape = cfg.shape
        R, L, nlp = cfg.ranks, cfg.ranks_per_node, cfg.slots_per_rank
        assert group.size() == R
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.placement, self.caps = plan_layer(cfg, sizing_routing, pool_routing, self.device, group)
        self.redos = 0
        self.gpu_plan = True
        self.c_num, self.c_den = c_rational(cfg.router_c)
        self._ccfg = make_cfg(cfg, self.caps, self.c_num, self.c_den)
        if _runtime is None:
            self._rt = Runtime(self.rank, R, self.device.index, LayerHandle.arena_bytes(self._ccfg))
            if R > 1:
                self._rt.exchange_handles(group)
            self._own_rt = True
        else:
            self._rt, self._own_rt = _runtime, False
        self._h = LayerHandle(self._rt, self._ccfg)
        self._h.set_placement(self.placement)
        self.w1 = self.w2 = None
        self._y = torch.empty(cfg.max_tokens_per_rank, shape.hidden, dtype=dtype, device=self.device)
        self._swap_moves = 0
        self._epoch = 0
        self._plan_views = None
        self._tokens = cfg.max_tokens_per_rank        # the bucket the next step runs at
        self._pad_bufs = {}

    @staticmethod
    def arena_bytes(cfg, caps):
        c_num, c_den = c_rational(cfg.router_c)
        return LayerHandle.arena_bytes(make_cfg(cfg, caps, c_num, c_den))

    # -- weights ------------------------------------------------------------------------
    def load_weights(self, w1_of, w2_of):
        """w1_of(e) -> [ffn1, H], w2_of(e) -> [H, ffn] for every expert this rank hosts; the pad group
        and unassigned redundant slots stay zero."""
        cfg, shape = self.cfg, self.cfg.shape
        nlp, gpe = cfg.slots_per_rank, cfg.groups_per_rank
        if cfg.swap:       # swapped experts travel between ranks: the layer's own peer-visible slots
            w1, w2 = self._h.weight_slots(gpe, shape.ffn1, shape.hidden, shape.ffn_hidden)
            w1.zero_()
            w2.zero_()
        else:
            w1 = torch.zeros(gpe, shape.ffn1, shape.hidden, dtype=self.dtype, device=self.device)
            w2 = torch.zeros(gpe, shape.hidden, shape.ffn_hidden, dtype=self.dtype, device=self.device)
        mine = self.placement.p2l[self.rank * nlp:(self.rank + 1) * nlp].tolist()
        for group_index, expert in enumerate(mine, start=1):          # group 0 is the pad group
            if expert >= 0:
                w1[group_index].copy_(w1_of(expert).to(self.dtype))
                w2[group_index].copy_(w2_of(expert).to(self.dtype))
        self.set_weights(w1, w2)

    def set_weights(self, w1_slots, w2_slots):
        """Per-group weights [gpe, ffn1, H] / [gpe, H, ffn]; the layer keeps references (no copy)."""
        shape, gpe = self.cfg.shape, self.cfg.groups_per_rank
        assert w1_slots.shape == (gpe, shape.ffn1, shape.hidden), tuple(w1_slots.shape)
        assert w2_slots.shape == (gpe, shape.hidden, shape.ffn_hidden), tuple(w2_slots.shape)
        self.w1, self.w2 = w1_slots.contiguous(), w2_slots.contiguous()
        torch.cuda.synchronize()
        self._h.set_weights(self.w1, self.w2)

    # -- setup ------------------------------------------------------------------------
    def prime(self, topk_ids, topk_weights):
        """One planning pass with every rank quiesced (loads kernels, checks the routing).  With swap on the pass
        is a whole step on zero tokens: the swap decision is part of planning, and the experts it moves travel
        inside the GEMM kernels of the same step, so a plan is always followed by its forward."""
        plan = self.prepare(topk_ids, topk_weights)
        if self.cfg.swap:
            self.forward(torch.zeros(self._tokens, self.cfg.shape.hidden, dtype=self.dtype, device=self.device), plan)
        self.check()
        self._barrier()
        return plan

    def _barrier(self):
        torch.cuda.synchronize()
        if self.cfg.ranks > 1 and not getattr(self.group, "is_local", False):
            torch.distributed.barrier(group=self.group)

    # -- per iteration ----------------------------------------------------------------------
    def _ids(self, topk_ids, topk_weights):
        ids = topk_ids.to(device=self.device, dtype=torch.int32).contiguous()
        wts = topk_weights.to(device=self.device, dtype=torch.float32).contiguous()
        assert ids.shape == (self._tokens, self.cfg.shape.topk), (tuple(ids.shape), self._tokens)
        return ids, wts

    # -- token buckets ----------------------------------------------------------------------
    def set_tokens(self, tokens):
        """Run the following steps at `tokens` rows per rank (<= max_tokens_per_rank; every rank must choose the
        same value, as the reference's ranks pad to a common bucket, python/zepp/serving.py:5-6).  Buffers keep
        their size; a step graph is captured per (bucket, tensors)."""
        tokens = int(tokens)
        if tokens != self._tokens:
            self._h.set_tokens(tokens)
            self._tokens = tokens
            self._plan_views = None

    def step_padded(self, topk_ids, topk_weights, x, bucket=None):
        """One step on n <= bucket real tokens: rows n..bucket-1 are pad rows (expert id -1: no owner, no transfer,
        no compute, not counted in the loads).  `bucket` defaults to the smallest of token_buckets(cfg) that holds n;
        every rank must pass the same bucket.  Returns y[:n].  The padded inputs live in per-bucket buffers, so a
        bucket's step graph is captured once."""
        n = int(topk_ids.shape[0])
        if bucket is None:
            bucket = next(b for b in token_buckets(self.cfg) if b >= n)
        assert n <= bucket <= self.cfg.max_tokens_per_rank, (n, bucket)
        K, H = self.cfg.shape.topk, self.cfg.shape.hidden
        if bucket not in self._pad_bufs:
            self._pad_bufs[bucket] = (torch.full((bucket, K), -1, dtype=torch.int32, device=self.device),
                                      torch.zeros(bucket, K, dtype=torch.float32, device=self.device),
                                      torch.zeros(bucket, H, dtype=self.dtype, device=self.device))
        ids_b, w_b, x_b = self._pad_bufs[bucket]
        ids_b[:n].copy_(topk_ids)
        ids_b[n:].fill_(-1)
        w_b[:n].copy_(topk_weights)
        x_b[:n].copy_(x)
        self.set_tokens(bucket)
        return self.step(ids_b, w_b, x_b)[:n]

    def prepare(self, topk_ids, topk_weights, marks=None, phase=None):
        """Loads exchange -> (swap decision) -> route -> routing exchange -> metadata; returns the Plan.
        With swap on, run forward() on this plan before the next prepare(): the weights of the experts a decision
        moves are pulled by the forward's GEMM kernels.
        `phase` (0..3) runs one stage only: ranks emulated inside one process advance in lock step.
        The id / weight tensors are read in place by the step's kernels (keep them unchanged until then)."""
        ids, wts = self._ids(topk_ids, topk_weights)
        self._keep = (ids, wts)
        if phase is None and marks is None:
            self._h.prepare(ids, wts)
        elif phase is None:
            self._h.prepare(ids, wts, 0)
            marks("plan_comm")
            self._h.prepare(ids, wts, 1)
            marks("place")
            self._h.prepare(ids, wts, 2)
            self._h.prepare(ids, wts, 3)
            marks("plan")
        else:
            self._h.prepare(ids, wts, phase)
            if phase < 3:
                return None
        self._epoch += 1
        if self._plan_views is None:          # runtime buffers: the addresses never change
            K = self.cfg.shape.topk
            self._plan_views = (self._h.table("vce").view(-1, K), self._h.table("probs_all").view(-1, K))
        return Plan(self._plan_views[0], self._plan_views[1], stable=True, epoch=self._epoch)

    def forward(self, x, plan=None, marks=None, phase=None):
        assert x.shape == (self._tokens, self.cfg.shape.hidden), (tuple(x.shape), self._tokens)
        x = x.contiguous()
        y = self._y[:self._tokens]
        if phase is not None:
            self._h.forward(x, y, phase)
            return y
        if marks is None:
            self._h.forward(x, y)
            return y
        self._h.forward(x, y, 0)
        self._h.forward(x, y, 1)
        marks("dispatch")
        marks("act")                     # the activation runs in the dispatch GEMM's epilogue
        self._h.forward(x, y, 2)
        self._h.forward(x, y, 3)
        marks("combine")
        return y

    def step(self, topk_ids, topk_weights, x):
        """prepare + forward in one runtime call (lowest host overhead)."""
        ids, wts = self._ids(topk_ids, topk_weights)
        self._keep = (ids, wts)
        assert x.shape == (self._tokens, self.cfg.shape.hidden), (tuple(x.shape), self._tokens)
        y = self._y[:self._tokens]
        self._h.step(ids, wts, x.contiguous(), y)
        self._epoch += 1
        return y

    # -- verdict ----------------------------------------------------------------------------
    def check(self):
        """Synchronise and raise if the last steps recorded a device-side error (a wait that ran out,
        a capacity violation, a bad index).  The reference checks capacities on the host before it
        launches (python/zepp/comm/overlap.py:136-145); here the verdict is deferred and read on demand."""
        st = self._h.status()
        if st[4]:
            dem = self._h.table("demands").cpu().tolist()
            d = Demands(*[int(v) for v in dem[:7]])
            raise CapacityExceeded(violations(d, self.caps, direct=self.cfg.comm_strategy == "direct"), d)
        if st[0]:
            what = ", ".join(n for b, n in _ERR_NAMES.items() if st[0] & b)
            raise RuntimeError(f"zepp_b200 step failed: {what} (wait id {st[1]}, peer/item {st[2]}, epoch {st[3]})")

    TRACE_NAMES = ("route", "pass1", "pass1_go", "pass2", "gemm1", "gemm1_x", "gemm1_end", "gemm2", "gemm2_end",
                   "reduce", "reduce_go", "reduce_end", "scan", "scan_counts", "scan_bases", "scan_demands",
                   "scan_sched", "scan_end", "loads", "decide", "decide_go", "decide_end", "gather_end", "first_items")
    # loads .. decide_end: the swap kernels that run before the routing (cycle counters in a profile build)

    def trace(self):
        """Device timeline of the last step: microseconds of each stamp after the step's first kernel."""
        t = self._h.trace()[8:8 + len(self.TRACE_NAMES)]
        t0 = t[0]
        return {n: (v - t0) / 1e3 if v else None for n, v in zip(self.TRACE_NAMES, t) if n is not None}

    def step_ring(self):
        """(start, end) device stamps in microseconds of the last 16 steps, oldest first, relative to the oldest start."""
        t = self._h.trace()
        pairs = sorted((t[32 + i], t[48 + i]) for i in range(16) if t[32 + i])
        if not pairs:
            return []
        t0 = pairs[0][0]
        return [((a - t0) / 1e3, (b - t0) / 1e3) for a, b in pairs]

    def tables(self, *names):
        """Planner products of the last prepare (device tensors): see runtime.TABLES."""
        return [self._h.table(n) for n in names]

    @property
    def gpu_launches(self):
        return self._h.launches()

    @property
    def swap_moves(self):
        """Expert moves of the last step's swap decision (reads the device result block: synchronises)."""
        if not self.cfg.swap:
            return 0
        return int(self._h.table("swap_block")[1])

    def current_placement(self):
        """The placement the device tables hold now (they change when a swap is decided)."""
        from .placement import Placement, rebuild_l2p
        p2l = self._h.table("p2l").cpu()
        return Placement(p2l, rebuild_l2p(p2l, self.cfg.shape.num_experts, self.cfg.ranks), self.placement.lcnts,
                         dict(self.placement.stats))

    def resize_capacities(self, demands=None, caps=None):
        """Collective: rebuild this rank's buffers for larger capacities (`caps`, or the growth rule applied to the
        `demands` of a step that raised CapacityExceeded -- they are identical on every rank), keeping the
        placement the device tables hold now and the weights.  The reference grows collectively and plans the step
        again (python/zepp/capacity.py:75-82, python/zepp/serving.py:434-451); callers repeat the step likewise."""
        assert self._own_rt, "layers that share a caller's runtime cannot be resized"
        from .capacity import grow
        torch.cuda.synchronize()
        if caps is None:
            caps = grow(self.caps, demands, direct=self.cfg.comm_strategy == "direct")
        cfg, shape = self.cfg, self.cfg.shape
        placement = self.current_placement()
        old_h, old_rt, w1, w2 = self._h, self._rt, self.w1, self.w2
        self._barrier()
        self.caps = caps
        self._ccfg = make_cfg(cfg, caps, self.c_num, self.c_den)
        self._rt = Runtime(self.rank, cfg.ranks, self.device.index, LayerHandle.arena_bytes(self._ccfg))
        if cfg.ranks > 1:
            self._rt.exchange_handles(self.group)
        self._h = LayerHandle(self._rt, self._ccfg)
        self._h.set_placement(placement)
        self.placement = placement
        if w1 is not None:
            if cfg.swap:       # the weights live in the old arena's slots: copy them into the new ones
                n1, n2 = self._h.weight_slots(cfg.groups_per_rank, shape.ffn1, shape.hidden, shape.ffn_hidden)
                n1.copy_(w1)
                n2.copy_(w2)
                w1, w2 = n1, n2
            self.set_weights(w1, w2)
        old_h.destroy()
        old_rt.destroy()
        self._plan_views = None
        tokens, self._tokens = self._tokens, cfg.max_tokens_per_rank
        self.set_tokens(tokens)
        self.redos += 1
        self._barrier()
        return caps

    def prep(self):
        """Per-iteration hygiene hook of the reference's benchmark loop: nothing to clear here (every
        buffer row that is read in a step is written in that step)."""
        return

    def close(self):
        self._h.destroy()
        if self._own_rt:
            self._rt.destroy()


def make_local_layers(cfg: EPMoEConfig, sizing_routing, pool_routing, wait_limit_ms=None):
    """All `cfg.ranks` ranks of a layer inside this process on the current GPU (their arenas are
    linked by plain pointers).  Kernels of different ranks never wait on one another this way as
    long as every rank finishes a phase before any rank starts the next: use `local_step`."""
    R = cfg.ranks
    dev = torch.device("cuda", torch.cuda.current_device())
    _, caps = plan_layer(cfg, sizing_routing, pool_routing, dev, None)
    nbytes = EPMoE.arena_bytes(cfg, caps)
    rts = [Runtime(r, R, dev.index, nbytes) for r in range(R)]
    if wait_limit_ms:
        for rt in rts:
            rt.set_wait_limit_ms(wait_limit_ms)
    Runtime.link_local(rts)
    return [EPMoE(cfg, LocalGroup(r, R), sizing_routing, pool_routing, _runtime=rts[r]) for r in range(R)], rts


def local_step(layers, ids_all, wts_all, xs):
    """One layer step of in-process ranks, phase by phase; returns the list of outputs."""
    for ph in range(4):
        for r, l in enumerate(layers):
            l.prepare(ids_all[r], wts_all[r], phase=ph)
    for ph in range(4):
        for r, l in enumerate(layers):
            l.forward(xs[r], phase=ph)
    return [l._y[:l._tokens] for l in layers]
