"""MoE-layer benchmark: one step = prepare (device planning) + forward (dispatch GEMM with SwiGLU,
combine GEMM, top-k reduce) of the expert-parallel layer on synthetic routing of a named workload.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference        # the reference layer math on the host cores (CPU arm)

Prints ONE JSON line on rank 0.  `value` = whole-job TFLOP/s (6*H*I flops per routed copy) with
inputs resident in HBM; `e2e` = the same through the public API with pinned host buffers copied
in and the output copied out inside the timed region; `roofline` = the dispatch GEMM kernel
against the measured HBM copy bandwidth; `cpu_baseline` = the CPU oracle layer on a bounded sample.
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

# dram__bytes_read.sum + dram__bytes_write.sum of one dispatch-GEMM launch from the ncu capture summarised in
# profiles/moe_gemm_qwen3-30b_1gpu.md, keyed by (workload, GPUs, tokens per rank)
NCU_TRAFFIC = {("qwen3-30b", 1, 512): 849.7e6}
METRIC = "moe_layer_tflops"
UNIT = "TFLOP/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen3-30b", choices=["qwen3-30b", "qwen3-235b", "k2"])
    ap.add_argument("--strategy", default="overlap", choices=["overlap", "direct"])
    ap.add_argument("--tokens", type=int, default=0, help="tokens per rank (default: the workload's)")
    ap.add_argument("--cpu-baseline", type=int, default=1)
    ap.add_argument("--trace-dir", default="", help="trace replay: draw the routing from this trace directory "
                    "(manifest.json + <model>/eval.txt, pool.txt) with the reference's batch sampler")
    ap.add_argument("--budget-mib", type=float, default=4.0, help="trace replay: send budget per rank (sets tokens/rank)")
    ap.add_argument("--swap", type=int, default=-1, help="expert swap on/off (default: the workload's setting)")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


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
    threads.  Returns (TFLOP/s, seconds per pass, threads)."""
    from oracle import layer as ol
    from zepp_b200 import workloads as wl
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    T = min(tokens, ids.shape[1])
    g = torch.Generator().manual_seed(777)
    E = shape.num_experts
    W1 = 0.02 * torch.randn(E, shape.ffn1, shape.hidden, generator=g)
    W2 = 0.02 * torch.randn(E, shape.hidden, shape.ffn_hidden, generator=g)
    x = wl.tokens(0, ids.shape[1], shape.hidden, seed=seed, dtype=torch.float32)[:T]
    i0, w0 = ids[0, :T], wts[0, :T]
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
    tf, sec, threads, T = cpu_reference_sample(shape, ids, wts, 0, max(args.steps, 3), warmup=min(max(args.warmup, 1), 5))
    line = {"impl": "reference", "metric": METRIC, "value": tf, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: H={shape.hidden} I={shape.ffn_hidden} E={shape.num_experts} "
                                   f"top-{shape.topk} SwiGLU, {S} tokens/rank", "sample": f"{T} tokens of rank 0 per step"},
            "cpu_baseline": {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": f"{T} tokens x top-{shape.topk}, fp32, all {shape.num_experts} experts resident"},
            "e2e": {"value": tf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    import torch.distributed as dist
    from zepp_b200 import EPMoE, EPMoEConfig
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

    if args.trace_dir:
        shape, S, ids, wts, pool_ids, trace_model = wl.from_trace(args.workload, world, args.trace_dir, args.budget_mib)
    else:
        shape, S, ids, wts, _, _ = wl.make(args.workload, world, S=args.tokens or None)
        pool_ids, trace_model = ids, None
    _, _, _, router_c, wl_swap = wl.WORKLOADS[args.workload]
    swap = bool(wl_swap if args.swap < 0 else args.swap) and args.strategy == "overlap" and world > 1
    cfg = EPMoEConfig(shape=shape, ranks=world, ranks_per_node=world, max_tokens_per_rank=S,
                      comm_strategy=args.strategy, swap=swap, router_c=router_c)
    layer = EPMoE(cfg, group, sizing_routing=ids, pool_routing=pool_ids)
    nlp = cfg.slots_per_rank
    hosted = [int(e) for e in layer.placement.p2l[rank * nlp:(rank + 1) * nlp].tolist() if e >= 0]
    wts_dev = wl.fast_weights(shape, hosted, dev)
    layer.load_weights(lambda e: wts_dev[e][0], lambda e: wts_dev[e][1])
    del wts_dev
    ids_own = ids[rank].contiguous()
    w_own = wts[rank].contiguous()
    ids_d, w_d = ids_own.to(dev), w_own.to(dev)
    n_x = 4
    xs_host = [wl.tokens(rank, S, shape.hidden, seed=s).pin_memory() for s in range(n_x)]
    xs_dev = [x.to(dev) for x in xs_host]
    ids_pin, w_pin = ids_own.pin_memory(), w_own.pin_memory()
    y_pin = torch.empty(S, shape.hidden, dtype=torch.bfloat16).pin_memory()
    layer.prime(ids_d, w_d)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731

    def step_resident(i, marks=None):
        if marks is None:
            return layer.step(ids_d, w_d, xs_dev[i % n_x])
        plan = layer.prepare(ids_d, w_d, marks)
        return layer.forward(xs_dev[i % n_x], plan, marks)

    # end-to-end path: every step copies its inputs from pinned host memory and its output back.  Two
    # buffer sets and two copy streams let the copies of neighbouring steps overlap the compute of this one
    # (each step still waits for its own inputs and delivers its own output).
    ids_in = [torch.empty_like(ids_d) for _ in range(2)]
    w_in = [torch.empty_like(w_d) for _ in range(2)]
    x_in = [torch.empty_like(xs_dev[0]) for _ in range(2)]
    y_dev = [torch.empty_like(xs_dev[0]) for _ in range(2)]
    y_pins = [y_pin, torch.empty_like(y_pin).pin_memory()]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    main = torch.cuda.current_stream()
    for e in ev_done:
        e.record(main)

    def step_e2e(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[b])               # step i-2 no longer reads this input set
            ids_in[b].copy_(ids_pin, non_blocking=True)
            w_in[b].copy_(w_pin, non_blocking=True)
            x_in[b].copy_(xs_host[i % n_x], non_blocking=True)
            ev_in[b].record(s_in)
        main.wait_event(ev_in[b])
        y = layer.step(ids_in[b], w_in[b], x_in[b])
        y_dev[b].copy_(y, non_blocking=True)
        ev_done[b].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[b])
            y_pins[b].copy_(y_dev[b], non_blocking=True)

    # ---- device-resident steps (value) + per-kernel brackets (roofline)
    for i in range(args.warmup):
        step_resident(i)
    layer.check()
    sampler = ClockSampler(local_rank)
    names = ("start", "plan_comm", "place", "plan", "dispatch", "act", "combine")
    launches0 = layer.gpu_launches
    sampler.start()                  # before the barrier: NVML start-up time differs per rank
    barrier()
    t_begin, t_end = ev(), ev()
    t_begin.record()
    h0 = time.perf_counter()
    for i in range(args.steps):
        step_resident(i)
    host_us = (time.perf_counter() - h0) / args.steps * 1e6      # host enqueue time per step (no sync inside)
    t_end.record()
    steady = layer.trace()           # device stamps of the last step of the timed loop (steady state)
    ring = layer.step_ring()
    barrier()
    launches = layer.gpu_launches - launches0
    layer.check()
    ms_total = max_over_ranks(t_begin.elapsed_time(t_end))
    ms_step = ms_total / args.steps
    for i in range(3):
        step_resident(i)
    timeline = layer.trace()         # device-side stamps of the last graph-launched step
    # per-kernel brackets (the reference's marks): the same steps again, phase by phase, events between
    evs = [{n: ev() for n in names} for _ in range(args.steps)]
    barrier()
    for i in range(args.steps):
        e = evs[i]
        e["start"].record()
        step_resident(i, lambda n, e=e: e[n].record())
    barrier()
    clocks = sampler.stop()
    gemm1_ms = statistics.mean(e["plan"].elapsed_time(e["dispatch"]) for e in evs)
    plan_ms = statistics.mean(e["start"].elapsed_time(e["plan"]) for e in evs)
    comb_ms = statistics.mean(e["act"].elapsed_time(e["combine"]) for e in evs)

    # ---- end-to-end steps through the public API with host buffers
    for i in range(max(3, args.warmup // 2)):
        step_e2e(i)
    barrier()
    t0, t1 = ev(), ev()
    t0.record()
    for i in range(args.steps):
        step_e2e(i)
    s_out.wait_stream(main)
    t1.record(s_out)                 # after the last output has landed in host memory
    barrier()
    ms_e2e = max_over_ranks(t0.elapsed_time(t1)) / args.steps
    layer.check()

    if world > 1:
        steady_all = [None] * world
        dist.all_gather_object(steady_all, {k: steady[k] for k in ("pass1", "pass1_go", "pass2", "gemm1", "gemm1_x",
                                                                   "gemm1_end", "gemm2", "gemm2_end", "reduce", "reduce_go",
                                                                   "reduce_end", "gather_end", "first_items")} | {"host_us": host_us})
    else:
        steady_all = [steady]
    # ---- roofline of the dispatch GEMM kernel (HBM bound at these row counts)
    H, I, K = shape.hidden, shape.ffn_hidden, shape.topk
    splits, m_this = layer.tables("splits", "m_this")
    gpe = cfg.groups_per_rank
    mine = splits[rank * gpe:(rank + 1) * gpe].cpu()
    active = int((mine > 0).sum())
    m_r = int(m_this[0])
    alg_bytes = 4.0 * H * I * active + 2.0 * H * m_r + 2.0 * I * m_r      # W1 of active experts + rows in + activations out
    hbm_gbs, bf16_tf, peak_kind = peaks()
    achieved = alg_bytes / (gemm1_ms * 1e-3) / 1e9
    flops_step = 6.0 * H * I * S * K * world
    value = flops_step / (ms_step * 1e-3) / 1e12
    e2e_val = flops_step / (ms_e2e * 1e-3) / 1e12
    t_flop = 6.0 * H * I * m_r / (bf16_tf * 1e12)
    t_hbm = 6.0 * H * I * active / (hbm_gbs * 1e9)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic" if not trace_model else f"routing replayed from trace slice '{trace_model}' "
                                                        f"({args.budget_mib} MiB budget); tokens and weights synthetic",
        "config": {"workload": f"{args.workload}: H={H} I={I} E={shape.num_experts} top-{K} SwiGLU, {S} tokens/rank, "
                               f"{shape.num_experts // world} experts/rank, "
                               + ("routing seed 0" if not trace_model else "trace-replay routing"),
                   "strategy": args.strategy, "parallelism": f"ep{world}", "router_c": router_c, "swap": int(swap),
                   "l2": "expert weights streamed per step exceed the 126 MB L2 (inputs larger than L2)",
                   "timed": "prepare (device planning) + forward"},
        "latency_us": ms_step * 1e3,
        "device_timeline_us": timeline,
        "host_enqueue_us_per_step": host_us,
        "last_steps_start_end_us": ring,
        "steady_timeline_us": steady_all,
        "breakdown_us": {"plan": plan_ms * 1e3, "dispatch_gemm": gemm1_ms * 1e3, "combine_gemm_reduce": comb_ms * 1e3},
        "roofline_layer": {"t_flop_us": t_flop * 1e6, "t_hbm_weights_us": t_hbm * 1e6,
                           "frac_of_3term": max(t_flop, t_hbm) / (ms_step * 1e-3), "rows_this_rank": m_r},
        "e2e": {"value": e2e_val, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(ids_pin.numel() * 4 + w_pin.numel() * 4 + xs_host[0].numel() * 2),
                "d2h_bytes_per_step": int(y_pin.numel() * 2),
                "pipelined": "inputs of step i+1 and the output of step i-1 are copied on side streams during step i"},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "kernel": "moe_gemm_kernel<gate|up + SwiGLU> (dispatch GEMM)", "achieved": achieved,
                     "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs, "peak_kind": peak_kind,
                     "traffic": NCU_TRAFFIC.get((args.workload, world, S)), "algorithmic_bytes": alg_bytes,
                     "kernel_ms": gemm1_ms,
                     "kernel_ms_device_stamps": (steady["gemm1_end"] - steady["gemm1"]) / 1e3 if steady.get("gemm1_end") else None},
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and args.cpu_baseline:
        tf, sec, threads, T = cpu_reference_sample(shape, ids, wts, 0, 10)
        line["cpu_baseline"] = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port", "ms_per_pass": sec * 1e3,
                                "sample": f"{T} tokens x top-{K} of rank 0, fp32, oracle/layer.py on all host threads"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    layer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
