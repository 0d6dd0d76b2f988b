"""MoE-layer benchmark: one step = prepare (device planning) + forward (dispatch GEMM with SwiGLU,
combine GEMM, top-k reduce) of the expert-parallel layer on synthetic routing of a named workload.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference        # the reference layer math on the host cores (CPU arm)
    python bench.py --sweep 1 [--gpus N]    # decode / prefill sweep: one JSON line per (tokens, routing, strategy)

Prints ONE JSON line on rank 0 (the sweep: one per point).  The default workload is the Qwen3-235B-A22B layer
shape with Zipf(1.0) routing, router_c 0.25 and expert swap on at more than one GPU; at 8 GPUs the same process
also measures the Qwen3-30B uniform case and the Kimi-K2 case with per-step popularity drift (fused and unfused
dispatch) and reports them under `extra_configs`.  `value` = whole-job TFLOP/s (6*H*I flops per routed copy)
with inputs resident in HBM; `e2e` = the same through the public API with pinned host buffers copied in and the
output copied out inside the timed region; `roofline` = the dispatch GEMM kernel against the measured HBM copy
bandwidth; `roofline_layer` = the step against max(FLOPs / bf16 peak, NVLink bytes / 900 GB/s) evaluated on the
step's own routing tables (and the same with the HBM weight term); `parity` = sampled tokens of one step against
the CPU oracle; `cpu_baseline` = the CPU oracle layer on a bounded sample.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# dram__bytes_read.sum + dram__bytes_write.sum of one dispatch-GEMM launch from an ncu capture of the same
# command, keyed by (workload, GPUs, tokens per rank)
NCU_TRAFFIC = {("qwen3-235b", 1, 512): 3310.6e6, ("qwen3-30b", 1, 512): 848.3e6}
METRIC = "moe_layer_tflops"
UNIT = "TFLOP/s"
NVLINK_BPS = 900e9            # per direction per GPU: the figure the roofline is defined with


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen3-235b", choices=["qwen3-30b", "qwen3-235b", "k2"])
    ap.add_argument("--strategy", default="overlap", choices=["overlap", "direct"])
    ap.add_argument("--tokens", type=int, default=0, help="tokens per rank (default: the workload's)")
    ap.add_argument("--cpu-baseline", type=int, default=1)
    ap.add_argument("--trace-dir", default="", help="trace replay: draw the routing from this trace directory "
                    "(manifest.json + <model>/eval.txt, pool.txt) with the reference's batch sampler")
    ap.add_argument("--budget-mib", type=float, default=4.0, help="trace replay: send budget per rank (sets tokens/rank)")
    ap.add_argument("--swap", type=int, default=-1, help="expert swap on/off (default: the workload's setting)")
    ap.add_argument("--extra", type=int, default=-1, help="also run the other 8-GPU configurations (default: at 8 GPUs)")
    ap.add_argument("--sweep", type=int, default=0, help="decode / prefill sweep on the qwen3-235b shape")
    ap.add_argument("--e2e-buffers", type=int, default=3, help="buffer sets of the end-to-end path (host copies in flight)")
    ap.add_argument("--parity-tokens", type=int, default=6, help="tokens of rank 0 checked against the CPU oracle")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), float(p.get("bf16_tflops_sustained", 1400.0)), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU through NVML (read-only) from a thread while
    the timed region runs."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index, period_s=0.002):
        self.index, self.period, self.sm, self.bits, self.max_mhz = index, period_s, [], 0, None
        self.stop_flag = threading.Event()
        self.thread = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = torch.cuda.get_device_properties(self.index).uuid
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:  # noqa: BLE001
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.nv = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            self.nv = None
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _sample(self):
        self.sm.append(float(self.nv.nvmlDeviceGetClockInfo(self.handle, self.nv.NVML_CLOCK_SM)))
        self.bits |= int(self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))

    def _loop(self):
        while not self.stop_flag.is_set():
            try:
                self._sample()
            except Exception:  # noqa: BLE001
                return
            time.sleep(self.period)

    def stop(self):
        if getattr(self, "nv", None) is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        try:
            self._sample()
        except Exception:  # noqa: BLE001
            pass
        reasons = [n for b, n in self.REASONS.items() if self.bits & b]
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.sm)}


def cpu_reference_sample(shape, ids, wts, seed, iters, tokens=128, warmup=2):
    """The reference's fp32 SwiGLU layer (oracle/layer.py) on the first `tokens` tokens of rank 0, all host
    threads.  Returns (TFLOP/s, seconds per pass, threads, tokens)."""
    from oracle import layer as ol
    from zepp_b200 import workloads as wl
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    T = min(tokens, ids.shape[1])
    g = torch.Generator().manual_seed(777)
    i0, w0 = ids[0, :T], wts[0, :T]
    touched = sorted(set(i0.reshape(-1).tolist()))
    W1 = {e: 0.02 * torch.randn(shape.ffn1, shape.hidden, generator=g) for e in touched}
    W2 = {e: 0.02 * torch.randn(shape.hidden, shape.ffn_hidden, generator=g) for e in touched}
    x = wl.tokens(0, ids.shape[1], shape.hidden, seed=seed, dtype=torch.float32)[:T]
    for _ in range(warmup):
        ol.moe_reference_fp32(x, i0, w0, W1, W2)
    ts = []
    for _ in range(iters):
        t0 = time.perf_counter()
        ol.moe_reference_fp32(x, i0, w0, W1, W2)
        ts.append(time.perf_counter() - t0)
    sec = statistics.median(ts)
    flops = 6.0 * shape.hidden * shape.ffn_hidden * T * shape.topk
    return flops / sec / 1e12, sec, threads, T


def run_reference(args, rank):
    """CPU arm: the reference's layer math on the host cores, same metric/unit/config."""
    if rank != 0:
        return
    from zepp_b200 import workloads as wl
    shape, S, ids, wts, _, _ = wl.make(args.workload, max(args.gpus, 1), S=args.tokens or None)
    tokens = 16 if shape.hidden * shape.ffn_hidden > 4e6 else 128     # about 10-30 s of CPU work per run
    tf, sec, threads, T = cpu_reference_sample(shape, ids, wts, 0, max(min(args.steps, 10), 3), tokens=tokens,
                                               warmup=min(max(args.warmup, 1), 3))
    line = {"impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: H={shape.hidden} I={shape.ffn_hidden} E={shape.num_experts} "
                                   f"top-{shape.topk} SwiGLU, {S} tokens/rank", "sample": f"{T} tokens of rank 0 per step"},
            "cpu_baseline": {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"{T} tokens x top-{shape.topk}, fp32, weights of the touched experts resident"},
            "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


class Ctx:
    """Process-wide state of one benchmark process (one rank)."""

    def __init__(self, rank, local_rank, world, dev, group, dist):
        self.rank, self.local_rank, self.world, self.dev, self.group, self.dist = rank, local_rank, world, dev, group, dist

    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, v):
        if self.world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def layer_roofline(shape, W, gpe, sps, uc, splits, hbm_gbs, bf16_tf):
    """The step's roofline terms from its own routing tables (identical on every rank), max over ranks:
    FLOPs_r = 6 H I m_r; NVLink bytes_r = 2H (max(out, in) dedup'ed dispatch rows + max(out, in) combine rows);
    HBM weight bytes_r = 6 H I (local experts with at least one row)."""
    H, I = shape.hidden, shape.ffn_hidden
    C = sps.reshape(W, W, gpe).sum(-1).double()              # C[s, d]: copies of source s computed on rank d
    u = uc[:, :W].double()                                   # u[s, d]: tokens of s with at least one copy on d
    act = (splits.reshape(W, gpe) > 0).sum(-1).double()
    rows = C.sum(0)
    t_flop = 6.0 * H * I * rows / (bf16_tf * 1e12)
    off = 1.0 - torch.eye(W, dtype=torch.float64)
    d_out, d_in = (u * off).sum(1), (u * off).sum(0)
    c_out, c_in = (C * off).sum(0), (C * off).sum(1)         # owner r returns C[:, r] rows; home r receives C[r, :]
    t_nvl = 2.0 * H * (torch.maximum(d_out, d_in) + torch.maximum(c_out, c_in)) / NVLINK_BPS
    t_hbm = 6.0 * H * I * act / (hbm_gbs * 1e9)
    two = torch.maximum(t_flop, t_nvl)
    three = torch.maximum(two, t_hbm)
    return {"t_flop_us": float(t_flop.max()) * 1e6, "t_nvlink_us": float(t_nvl.max()) * 1e6,
            "t_hbm_weights_us": float(t_hbm.max()) * 1e6, "t_roof_2term_us": float(two.max()) * 1e6,
            "t_roof_3term_us": float(three.max()) * 1e6, "rows_max": int(rows.max()), "rows_min": int(rows.min()),
            "dispatch_rows_out_in_max": [int(d_out.max()), int(d_in.max())],
            "combine_rows_out_in_max": [int(c_out.max()), int(c_in.max())]}


def run_case(ctx, args, workload, strategy, tokens=None, swap=None, drift_steps=0, steps=32, warmup=5, zipf=None,
             want_e2e=True, want_brackets=False, max_tokens=None, pad_to=None, layer_cache=None):
    """Build the layer for one configuration, time `steps` steps (device-resident inputs), optionally the end-to-end
    path and the per-kernel brackets, check sampled tokens against the oracle.  Returns a dict (same on every rank
    for the timed numbers).  `pad_to`: run `tokens` real tokens inside a bucket of `pad_to` rows."""
    from oracle import layer as ol
    from zepp_b200 import EPMoE, EPMoEConfig
    from zepp_b200 import workloads as wl
    from zepp_b200.capacity import CapacityExceeded
    rank, world, dev = ctx.rank, ctx.world, ctx.dev
    key, S0, wl_zipf, router_c, wl_swap = wl.WORKLOADS[workload]
    shape = wl.shape_of(workload)
    S_real = tokens or S0
    S = pad_to or S_real                          # rows per rank a step runs at
    S_max = max_tokens or S
    zipf_s = wl_zipf if zipf is None else zipf
    swap_on = bool(wl_swap if swap is None else swap) and strategy == "overlap" and world > 1
    gen = torch.Generator().manual_seed(0)
    p = wl.popularity(shape.num_experts, zipf_s, gen)
    n_batches = max(1, drift_steps)
    batches, pool = [], None
    if args.trace_dir and tokens is None:
        # trace replay: the reference sampler's batch of this (slice, ranks, budget) and its pool window
        _, S_real, ids_b, wts_b, pool, _ = wl.from_trace(workload, world, args.trace_dir, args.budget_mib)
        S = S_max = S_real
        n_batches = 1
        batches.append((ids_b, wts_b))
    for b in range(n_batches - len(batches)):
        if b:
            p = wl.drift(p, 0.1, gen)
        ids_b, wts_b = wl.routing(world, S_max, shape.topk, p, gen)
        batches.append((ids_b, wts_b))
    cache_key = (workload, strategy, swap_on, S_max, zipf_s)
    if layer_cache is not None and cache_key in layer_cache:
        layer, cfg = layer_cache[cache_key]
    else:
        cfg = EPMoEConfig(shape=shape, ranks=world, ranks_per_node=world, max_tokens_per_rank=S_max,
                          comm_strategy=strategy, swap=swap_on, router_c=router_c)
        layer = EPMoE(cfg, ctx.group, sizing_routing=batches[0][0], pool_routing=batches[0][0] if pool is None else pool)
        layer.load_weights(lambda e: wl.device_expert(e, shape, dev)[0], lambda e: wl.device_expert(e, shape, dev)[1])
        if layer_cache is not None:
            layer_cache[cache_key] = (layer, cfg)
    layer.set_tokens(S)
    K, H, I = shape.topk, shape.hidden, shape.ffn_hidden

    def cut(t, fill):
        t = t[rank, :S].clone()
        t[S_real:] = fill
        return t.contiguous()

    ids_host = [cut(b[0], -1) for b in batches]
    w_host = [cut(b[1], 0.0) for b in batches]
    ids_d = [t.to(dev) for t in ids_host]
    w_d = [t.to(dev) for t in w_host]
    n_x = 4
    xs_host = [wl.tokens(rank, S_max, H, seed=s)[:S].contiguous().pin_memory() for s in range(n_x)]
    xs_dev = [x.to(dev) for x in xs_host]

    def step_resident(i, marks=None):
        b = i % n_batches
        if marks is None:
            return layer.step(ids_d[b], w_d[b], xs_dev[i % n_x])
        plan = layer.prepare(ids_d[b], w_d[b], marks)
        return layer.forward(xs_dev[i % n_x], plan, marks)

    # ---- dry pass over every batch: grow the buffers where a drifted batch needs it (collective, identical verdicts)
    redos0 = layer.redos
    for attempt in range(4):
        try:
            for i in range(max(n_batches, warmup, n_x)):          # every (batch, x buffer) pair: all step graphs captured
                step_resident(i)
                if i < n_batches:
                    layer.check()           # the verdict of every distinct batch (a later step overwrites the mask)
            layer.check()
            break
        except CapacityExceeded as e:
            layer.resize_capacities(e.demands)
            layer.set_tokens(S)
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    launches0 = layer.gpu_launches
    ctx.barrier()
    t_begin, t_end = ev(), ev()
    t_begin.record()
    h0 = time.perf_counter()
    for i in range(steps):
        step_resident(i)
    host_us = (time.perf_counter() - h0) / steps * 1e6       # host enqueue time per step (no sync inside)
    t_end.record()
    steady = layer.trace()           # device stamps of the last step of the timed loop (steady state)
    ring = layer.step_ring()
    ctx.barrier()
    launches = layer.gpu_launches - launches0
    layer.check()
    ms_step = ctx.max_over_ranks(t_begin.elapsed_time(t_end)) / steps
    starts = [a for a, _ in ring]
    period = statistics.median([b - a for a, b in zip(starts, starts[1:])]) if len(starts) > 2 else None
    period = ctx.max_over_ranks(period) if period is not None else None
    out = {"workload": workload, "strategy": strategy, "swap": int(swap_on), "tokens_per_rank": S_real, "bucket": S,
           "zipf": zipf_s, "router_c": router_c, "drift_batches": n_batches, "latency_us": ms_step * 1e3,
           "median_step_period_us": period, "gpu_launches_per_step": launches / steps,
           "host_enqueue_us_per_step": host_us, "capacity_redos": layer.redos - redos0,
           "timed": "mean over back-to-back graph-launched steps (prepare + forward), CUDA events, max over ranks; "
                    "median_step_period_us = median distance of the steps' device start stamps"}
    flops_step = 6.0 * H * I * S_real * K * world
    out["tflops"] = flops_step / (ms_step * 1e-3) / 1e12

    # ---- parity of one more step against the CPU oracle on sampled tokens of this rank (outside every timed region)
    xb = 1
    y = layer.step(ids_d[0], w_d[0], xs_dev[xb]).float().cpu()
    layer.check()
    n_par = min(args.parity_tokens, S_real)
    sample = torch.unique(torch.linspace(0, S_real - 1, n_par).long())
    ids_s, w_s, x_s = ids_host[0][sample], w_host[0][sample], xs_host[xb][sample]
    touched = sorted({int(e) for e in ids_s.reshape(-1).tolist() if e >= 0})
    W1, W2 = {}, {}
    for e in touched:
        a, b2 = wl.device_expert(e, shape, dev)
        W1[e], W2[e] = a.cpu(), b2.cpu()
    ref = ol.moe_reference_fp32(x_s, ids_s, w_s, W1, W2)
    refb = ol.moe_reference_bf16_points(x_s, ids_s, w_s, W1, W2).float()
    ys = y[sample]
    err = float((ys - ref).abs().max())
    scale = float(refb.abs().max())
    ok = bool(torch.allclose(ys, ref, rtol=2e-2, atol=2e-2)) and float((ys - refb).abs().max()) <= 1.5e-2 * scale
    del W1, W2
    flag = torch.tensor([0 if ok else 1], device=dev)
    worst = torch.tensor([err], dtype=torch.float64, device=dev)
    if world > 1:
        ctx.dist.all_reduce(flag)
        ctx.dist.all_reduce(worst, op=ctx.dist.ReduceOp.MAX)
    out["parity"] = {"ok": int(flag) == 0, "max_abs_err": float(worst), "tokens_per_rank_checked": int(sample.numel()),
                     "ranks_checked": world, "oracle": "oracle/layer.py fp32 path at rtol/atol 2e-2 and its bf16 path at "
                     "1.5 % of the largest reference magnitude", "ref_max_abs": scale}

    # ---- roofline of the step from its own tables (the parity step: batch 0 on the placement the run ended with)
    hbm_gbs, bf16_tf, bf16_sus, peak_kind = peaks()
    gpe = cfg.groups_per_rank
    splits, sps, uc, m_this = [t.cpu() for t in layer.tables("splits", "sps", "uc", "m_this")]
    rl = layer_roofline(shape, world, gpe, sps.reshape(world, -1), uc.reshape(world, -1), splits, hbm_gbs, bf16_tf)
    rl["frac_of_baseline_roofline"] = rl["t_roof_2term_us"] / (ms_step * 1e3)
    rl["frac_of_3term"] = rl["t_roof_3term_us"] / (ms_step * 1e3)
    rl["peaks"] = {"bf16_tflops": bf16_tf, "bf16_tflops_sustained": bf16_sus, "hbm_gbs": hbm_gbs,
                   "nvlink_gbs_per_direction": NVLINK_BPS / 1e9, "kind": peak_kind}
    out["roofline_layer"] = rl
    if world > 1:
        keys = ("pass1", "pass1_go", "pass2", "gemm1", "gemm1_x", "gemm1_end", "gemm2", "gemm2_end", "reduce",
                "reduce_go", "reduce_end", "gather_end", "first_items", "scan_end", "loads", "decide", "decide_go", "decide_end")
        steady_all = [None] * world
        ctx.dist.all_gather_object(steady_all, {k: steady.get(k) for k in keys})
        slow = max(range(world), key=lambda r: steady_all[r].get("gemm2_end") or 0)
        out["steady_timeline_us_slowest_rank"] = dict(steady_all[slow], rank=slow)
        out["steady_timeline_us_all_ranks"] = [{k: (round(v, 1) if v is not None else None) for k, v in d.items()}
                                               for d in steady_all]
    else:
        out["steady_timeline_us_slowest_rank"] = dict(steady, rank=0)
    out["_internal"] = {"layer": layer, "cfg": cfg, "ids_host": ids_host, "w_host": w_host, "xs_host": xs_host,
                        "step_resident": step_resident, "splits": splits, "m_this": m_this, "shape": shape, "S": S,
                        "n_batches": n_batches}
    return out


def run_e2e(ctx, case, steps, warmup, n_buf=3):
    """The same steps through the public API with HOST buffers: every step copies its inputs (ids, gate weights, x: one
    pinned block, one copy) from pinned host memory and its output back.  `n_buf` buffer sets and two copy streams let
    the copies of neighbouring steps overlap the compute of this one (each step still waits for its own inputs and
    delivers its own output)."""
    it = case["_internal"]
    layer, S, n_batches = it["layer"], it["S"], it["n_batches"]
    dev = ctx.dev
    xs_host = it["xs_host"]
    n_x = len(xs_host)
    K = it["ids_host"][0].shape[1]
    H = xs_host[0].shape[1]
    n_ids, n_w, n_xb = S * K * 4, S * K * 4, S * H * 2
    blob_bytes = n_ids + n_w + n_xb

    def views(blob):
        return (blob[:n_ids].view(torch.int32).view(S, K), blob[n_ids:n_ids + n_w].view(torch.float32).view(S, K),
                blob[n_ids + n_w:].view(torch.bfloat16).view(S, H))

    # host side: one pinned block per (batch, x buffer) pair the steps cycle through
    n_host = n_batches * n_x // __import__("math").gcd(n_batches, n_x)
    host_blobs = []
    for i in range(n_host):
        hb = torch.empty(blob_bytes, dtype=torch.uint8).pin_memory()
        hi, hw, hx = views(hb)
        hi.copy_(it["ids_host"][i % n_batches])
        hw.copy_(it["w_host"][i % n_batches])
        hx.copy_(xs_host[i % n_x])
        host_blobs.append(hb)
    dev_blobs = [torch.empty(blob_bytes, dtype=torch.uint8, device=dev) for _ in range(n_buf)]
    dev_views = [views(b) for b in dev_blobs]
    y_dev = [torch.empty(S, H, dtype=torch.bfloat16, device=dev) for _ in range(n_buf)]
    y_pins = [torch.empty(S, H, dtype=torch.bfloat16).pin_memory() for _ in range(n_buf)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(n_buf)]
    ev_done = [torch.cuda.Event() for _ in range(n_buf)]
    ev_out = [torch.cuda.Event() for _ in range(n_buf)]
    main = torch.cuda.current_stream()
    for e in ev_done + ev_out:
        e.record(main)

    def step_e2e(i):
        b = i % n_buf
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[b])               # the step that last used this input set has finished
            dev_blobs[b].copy_(host_blobs[i % n_host], non_blocking=True)
            ev_in[b].record(s_in)
        main.wait_event(ev_in[b])
        main.wait_event(ev_out[b])                    # its output set has been read out
        ids_b, w_b, x_b = dev_views[b]
        y = layer.step(ids_b, w_b, x_b)
        y_dev[b].copy_(y, non_blocking=True)
        ev_done[b].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[b])
            y_pins[b].copy_(y_dev[b], non_blocking=True)
            ev_out[b].record(s_out)

    for i in range(max(3, warmup // 2)):
        step_e2e(i)
    ctx.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(steps):
        step_e2e(i)
    s_out.wait_stream(main)
    t1.record(s_out)                 # after the last output has landed in host memory
    ctx.barrier()
    ms = ctx.max_over_ranks(t0.elapsed_time(t1)) / steps
    layer.check()
    # the same host <-> device copies alone (no step between them): what the host links deliver when every rank of
    # the box copies at once -- the floor of the end-to-end step time
    ctx.barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for i in range(steps):
        b = i % n_buf
        with torch.cuda.stream(s_in):
            dev_blobs[b].copy_(host_blobs[i % n_host], non_blocking=True)
        with torch.cuda.stream(s_out):
            y_pins[b].copy_(y_dev[b], non_blocking=True)
    main.wait_stream(s_in)
    main.wait_stream(s_out)
    c1.record()
    ctx.barrier()
    ms_copy = ctx.max_over_ranks(c0.elapsed_time(c1)) / steps
    return ms, int(blob_bytes), int(y_pins[0].numel() * 2), ms_copy


def run_brackets(ctx, case, steps):
    """Per-kernel brackets (the reference's marks): the same steps again, phase by phase, events between."""
    it = case["_internal"]
    names = ("start", "plan_comm", "place", "plan", "dispatch", "act", "combine")
    evs = [{n: torch.cuda.Event(enable_timing=True) for n in names} for _ in range(steps)]
    ctx.barrier()
    for i in range(steps):
        e = evs[i]
        e["start"].record()
        it["step_resident"](i, lambda n, e=e: e[n].record())
    ctx.barrier()
    it["layer"].check()
    return {"plan": statistics.mean(e["start"].elapsed_time(e["plan"]) for e in evs) * 1e3,
            "dispatch_gemm": statistics.mean(e["plan"].elapsed_time(e["dispatch"]) for e in evs) * 1e3,
            "combine_gemm_reduce": statistics.mean(e["act"].elapsed_time(e["combine"]) for e in evs) * 1e3}


def public(case):
    return {k: v for k, v in case.items() if k != "_internal"}


def close_case(case):
    case["_internal"]["layer"].close()
    case.pop("_internal")
    torch.cuda.empty_cache()


def run_sweep(ctx, args):
    """Decode / prefill sweep on the Qwen3-235B shape: tokens per rank 1 ... 4096 (token buckets of one layer sized
    for 4096; 1 token runs as one real row in the 8-row bucket), uniform and Zipf(1.0) routing, fused and unfused
    dispatch.  One JSON line per point on rank 0."""
    points = (1, 8, 32, 128, 512, 2048, 4096)
    for zipf in (0.0, 1.0):
        for strategy in ("overlap", "direct"):
            cache = {}
            for S in points:
                steps = 40 if S <= 512 else 12
                c = run_case(ctx, args, "qwen3-235b", strategy, tokens=S, swap=0, steps=steps, warmup=3, zipf=zipf,
                             max_tokens=4096, pad_to=max(S, 8), layer_cache=cache)
                if ctx.rank == 0:
                    rl = c["roofline_layer"]
                    print(json.dumps({"sweep": "config4", "n_gpus": ctx.world, "tokens_per_rank": S, "bucket": c["bucket"],
                                      "routing": "zipf1.0" if zipf else "uniform", "strategy": strategy,
                                      "latency_us": c["latency_us"], "tflops": c["tflops"],
                                      "t_roof_2term_us": rl["t_roof_2term_us"], "t_roof_3term_us": rl["t_roof_3term_us"],
                                      "frac_of_baseline_roofline": rl["frac_of_baseline_roofline"],
                                      "frac_of_3term": rl["frac_of_3term"], "parity_ok": c["parity"]["ok"],
                                      "gpu_launches_per_step": c["gpu_launches_per_step"]}), flush=True)
                if not c["parity"]["ok"]:
                    raise SystemExit(f"sweep point S={S} {strategy} zipf={zipf}: parity failed {c['parity']}")
                c.pop("_internal")
            for layer, _cfg in cache.values():
                layer.close()
            cache.clear()
            torch.cuda.empty_cache()


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    import torch.distributed as dist
    from zepp_b200 import workloads as wl
    from zepp_b200.layer import LocalGroup

    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE {world} (launch with torch.distributed.run)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        group = dist.group.WORLD
    else:
        group = LocalGroup(0, 1)
    ctx = Ctx(rank, local_rank, world, dev, group, dist)
    if args.sweep:
        run_sweep(ctx, args)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    sampler = ClockSampler(local_rank)
    sampler.start()                  # before the first barrier: NVML start-up time differs per rank
    swap = None if args.swap < 0 else args.swap
    drift = 16 if args.workload == "k2" else 0
    case = run_case(ctx, args, args.workload, args.strategy, tokens=args.tokens or None, swap=swap, drift_steps=drift,
                    steps=args.steps, warmup=args.warmup)
    br = run_brackets(ctx, case, min(args.steps, 16))
    clocks = sampler.stop()
    ms_e2e, h2d, d2h, ms_copy = run_e2e(ctx, case, args.steps, args.warmup, n_buf=args.e2e_buffers)
    it = case["_internal"]
    shape, S, cfg = it["shape"], it["S"], it["cfg"]
    H, I, K = shape.hidden, shape.ffn_hidden, shape.topk
    gpe = cfg.groups_per_rank
    mine = it["splits"][rank * gpe:(rank + 1) * gpe]
    active = int((mine > 0).sum())
    m_r = int(it["m_this"][0])
    # ---- roofline of the dispatch GEMM kernel (HBM bound at these row counts): W1 of the active experts once,
    #      routed rows in, activations out
    alg_bytes = 4.0 * H * I * active + 2.0 * H * m_r + 2.0 * I * m_r
    hbm_gbs, bf16_tf, _, peak_kind = peaks()
    gemm1_ms = br["dispatch_gemm"] / 1e3
    achieved = alg_bytes / (gemm1_ms * 1e-3) / 1e9
    flops_step = 6.0 * H * I * S * K * world
    ms_step = case["latency_us"] / 1e3
    steady = case["steady_timeline_us_slowest_rank"]
    line = {
        "metric": METRIC, "value": case["tflops"], "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic" if not args.trace_dir else f"routing replayed from the trace directory ({args.budget_mib} MiB "
                                                          "budget); tokens and weights synthetic",
        "config": {"workload": f"{args.workload}: H={H} I={I} E={shape.num_experts} top-{K} SwiGLU, {S} tokens/rank, "
                               f"{shape.num_experts // world} experts/rank, Zipf({case['zipf']}) routing seed 0"
                               + (f", {case['drift_batches']} drifting batches" if case["drift_batches"] > 1 else ""),
                   "strategy": args.strategy, "parallelism": f"ep{world}", "router_c": case["router_c"],
                   "swap": case["swap"],
                   "l2": "expert weights streamed per step exceed the 126 MB L2 (inputs larger than L2)",
                   "timed": case["timed"]},
        "latency_us": case["latency_us"],
        "median_step_period_us": case["median_step_period_us"],
        "host_enqueue_us_per_step": case["host_enqueue_us_per_step"],
        "steady_timeline_us_slowest_rank": steady,
        "steady_timeline_us_all_ranks": case.get("steady_timeline_us_all_ranks"),
        "breakdown_us": br,
        "roofline_layer": case["roofline_layer"],
        "parity": case["parity"],
        "capacity_redos": case["capacity_redos"],
        "e2e": {"value": flops_step / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "copies_alone_ms_per_step": ms_copy,
                "pipelined": f"{args.e2e_buffers} buffer sets: inputs of later steps and outputs of earlier ones are copied on side "
                             "streams during a step"},
        "gpu_launches": int(round(case["gpu_launches_per_step"] * args.steps)),
        "roofline": {"bound": "hbm", "kernel": "moe_gemm_kernel<gate|up + SwiGLU> (dispatch GEMM)", "achieved": achieved,
                     "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs, "peak_kind": peak_kind,
                     "traffic": NCU_TRAFFIC.get((args.workload, world, S)), "algorithmic_bytes": alg_bytes,
                     "kernel_ms": gemm1_ms, "rows_this_rank": m_r, "active_experts_this_rank": active,
                     "note": "rank 0's launch; at more than one GPU the kernel also waits for peers' rows, so the "
                             "HBM fraction is a lower bound there"},
        "clocks": clocks,
    }
    ok = case["parity"]["ok"]
    close_case(case)
    extra = args.extra if args.extra >= 0 else int(world == 8 and args.workload == "qwen3-235b" and not args.tokens)
    if extra:
        # the other 8-GPU configurations in the same process: latency and both roofline fractions each
        others = []
        for wname, strat, dr in (("qwen3-30b", "overlap", 0), ("k2", "overlap", 16), ("k2", "direct", 16)):
            c = run_case(ctx, args, wname, strat, drift_steps=dr, steps=max(dr, min(args.steps, 32)), warmup=args.warmup)
            ok = ok and c["parity"]["ok"]
            close_case(c)
            others.append(c)
        line["extra_configs"] = others
    if rank == 0 and world == 1 and args.cpu_baseline:
        _, _, ids, wts, _, _ = wl.make(args.workload, 1, S=args.tokens or None)
        tokens = 16 if H * I > 4e6 else 128
        tf, sec, threads, T = cpu_reference_sample(shape, ids, wts, 0, 5, tokens=tokens)
        line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "ms_per_pass": sec * 1e3,
                                "sample": f"{T} tokens x top-{K} of rank 0, fp32, oracle/layer.py on all host threads"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        sys.exit(3)                  # the layer's output left the oracle's tolerance: the numbers above do not count


if __name__ == "__main__":
    main()
