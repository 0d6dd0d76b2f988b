"""Loader of libzepp_b200.so and a thin tensor-level wrapper `C` whose function names follow the
reference's pybind module `zepp._C` (src/pybind/routing.cc:9-78, dispatch.cc:115-193) for the
stand-alone planner entry points.  There is no CPU fallback: a missing library raises."""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libzepp_b200.so")

SYMBOLS = (
    "zepp_last_error", "zepp_abi_version", "zepp_rt_create", "zepp_rt_destroy", "zepp_rt_ipc_handle",
    "zepp_rt_open_peers", "zepp_rt_link_local", "zepp_rt_set_wait_limit_ms", "zepp_rt_sm_count",
    "zepp_layer_arena_bytes", "zepp_layer_create", "zepp_layer_destroy", "zepp_layer_set_placement",
    "zepp_layer_set_weights", "zepp_layer_set_tokens", "zepp_layer_weight_slots", "zepp_layer_prepare", "zepp_layer_prepare_phase", "zepp_layer_forward",
    "zepp_layer_forward_phase", "zepp_layer_step", "zepp_layer_status", "zepp_layer_trace", "zepp_layer_table", "zepp_layer_gpu_launches",
    "zepp_route_workspace_ints", "zepp_route_ws_offsets", "zepp_route", "zepp_meta_workspace_bytes",
    "zepp_routed_meta", "zepp_routed_meta_noalloc", "zepp_dispatch_plan_words", "zepp_swap_decide_out_ints", "zepp_swap_decide",
    "zepp_lane_arm", "zepp_wait_geq",
)


class LayerCfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "num_experts", "topk", "hidden", "ffn_hidden", "act", "ranks", "ranks_per_node", "max_tokens_per_rank",
        "strategy", "swap", "redundant_slots_per_rank", "sm_margin", "gpu_plan")] + [
        ("_pad", ctypes.c_int32), ("c_num", ctypes.c_int64), ("c_den", ctypes.c_int64), ("caps", ctypes.c_int64 * 8)]


_lib = None


def lib():
    """The loaded shared library (raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m zepp_b200.build` "
                               "(there is no CPU fallback)")
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.zepp_last_error.restype = ctypes.c_char_p
        _lib.zepp_layer_arena_bytes.restype = ctypes.c_size_t
        _lib.zepp_meta_workspace_bytes.restype = ctypes.c_size_t
        _lib.zepp_rt_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_size_t,
                                        ctypes.POINTER(ctypes.c_void_p)]
    return _lib


def check(rc):
    if rc != 0:
        raise RuntimeError("zepp_b200: " + lib().zepp_last_error().decode())


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev_i32(t):
    assert t.is_cuda and t.dtype == torch.int32 and t.is_contiguous(), (t.device, t.dtype)
    return t


class _C:
    """Tensor-level entry points named after the reference's `zepp._C` functions."""

    def route_workspace_ints(self, G, R):
        return lib().zepp_route_workspace_ints(int(G), int(R))

    def route_ws_offsets(self, G, R):
        o = (ctypes.c_int64 * 10)()
        lib().zepp_route_ws_offsets(int(G), int(R), o)
        names = ("rep", "rphys", "c", "D", "U", "Lb", "fill", "M", "release", "extra")
        return dict(zip(names, (int(v) for v in o)))

    def route_fused(self, topk_own, loads, l2p, lcnts, my_rank, nlp, L, c_num, c_den, ws, probs_own=None, send=None):
        """Tables, budgets, deterministic assignment, vacate and (optionally) the send row of one rank.
        Returns (phys_own [S, K] int32, stats int64[4])."""
        S, K = topk_own.shape
        R, G = loads.shape
        phys = torch.empty(S, K, dtype=torch.int32, device=topk_own.device)
        stats = torch.zeros(4, dtype=torch.int64, device=topk_own.device)
        check(lib().zepp_route(_p(_dev_i32(topk_own)), S, K, _p(_dev_i32(loads)), _p(_dev_i32(l2p)), _p(_dev_i32(lcnts)),
                               G, R, int(my_rank), int(nlp), int(L), ctypes.c_int64(c_num), ctypes.c_int64(c_den),
                               _p(ws), _p(probs_own), _p(send), _p(phys), _p(stats), _stream()))
        return phys, stats

    route = route_fused

    def route_tables_only(self, loads, l2p, lcnts, my_rank, nlp, L, c_num, c_den, ws):
        R, G = loads.shape
        check(lib().zepp_route(_p(None), 0, 1, _p(_dev_i32(loads)), _p(_dev_i32(l2p)), _p(_dev_i32(lcnts)), G, R,
                               int(my_rank), int(nlp), int(L), ctypes.c_int64(c_num), ctypes.c_int64(c_den), _p(ws),
                               _p(None), _p(None), _p(None), _p(None), _stream()))

    def routed_meta_full(self, R, L, S, K, nlp, gpe, gathered=None, vce=None, my_rank=0, direct=False,
                         relay_slots=2, caps=None, copies_per_rank=None):
        """planner tail + routed metadata + demands + plan heads.  Returns a dict of device tensors."""
        dev = (gathered if gathered is not None else vce).device
        NN = R // L
        E = R * gpe
        n = R * S * K
        out = dict(
            vce=torch.empty(R * S, K, dtype=torch.int32, device=dev),
            probs_all=torch.empty(R * S, K, dtype=torch.float32, device=dev) if gathered is not None else None,
            splits=torch.empty(E, dtype=torch.int32, device=dev),
            scatter_index=torch.empty(R * S, K, dtype=torch.int32, device=dev),
            sps=torch.empty(R, E, dtype=torch.int32, device=dev),
            uc=torch.empty(R, R + NN, dtype=torch.int32, device=dev),
            demands=torch.zeros(8, dtype=torch.int64, device=dev),
            dplan=torch.zeros(lib().zepp_dispatch_plan_words(L, NN), dtype=torch.int64, device=dev),
            cplan=torch.zeros(4 * R + 2, dtype=torch.int64, device=dev) if NN == 1 else None,
        )
        caps_arr = (ctypes.c_int64 * 8)(*([1 << 40] * 8 if caps is None else [int(c) for c in caps]))
        ws = torch.empty(lib().zepp_meta_workspace_bytes(R, S, K, gpe), dtype=torch.uint8, device=dev)
        vin = None if vce is None else _dev_i32(vce.reshape(-1))
        check(lib().zepp_routed_meta(_p(gathered), _p(vin), R, L, S, K, int(nlp), int(gpe), int(my_rank), int(direct),
                                     int(relay_slots), caps_arr, int(S * K if copies_per_rank is None else copies_per_rank),
                                     _p(out["vce"]), _p(out["probs_all"]), _p(out["splits"]), _p(out["scatter_index"]),
                                     _p(out["sps"]), _p(out["uc"]), _p(out["demands"]), _p(out["dplan"]),
                                     _p(out["cplan"]), _p(ws), _stream()))
        assert n == out["vce"].numel()
        return out

    def routed_meta(self, vce, W, L, gpe):
        """(splits, scatter_index, sps, uc) of a virtual routing vce [W*S, K]."""
        S = vce.shape[0] // W
        o = self.routed_meta_full(W, L, S, vce.shape[1], gpe - 1, gpe, vce=vce.contiguous())
        return o["splits"], o["scatter_index"], o["sps"], o["uc"]

    def swap_decide_out_ints(self, R, G, nlp, cap):
        return lib().zepp_swap_decide_out_ints(int(R), int(G), int(nlp), int(cap))

    def swap_decide(self, loads, p2l, l2p, lcnts, L, nlp, C, cap, max_rounds, out):
        R, G = loads.shape
        check(lib().zepp_swap_decide(_p(_dev_i32(loads)), _p(_dev_i32(p2l)), _p(_dev_i32(l2p)), _p(_dev_i32(lcnts)), R, G,
                                     int(L), int(nlp), ctypes.c_double(C), int(cap), int(max_rounds), _p(out), _stream()))

    def lane_arm(self, out, R, rank, nlp, cap, gate, sched, ovr0, ovr1, stag, epoch):
        check(lib().zepp_lane_arm(_p(out), int(R), int(rank), int(nlp), int(cap), _p(gate), _p(sched), _p(ovr0),
                                  _p(ovr1), _p(stag), ctypes.c_int64(epoch), _stream()))

    def wait_geq(self, flag, value, limit_ms):
        res = torch.zeros(1, dtype=torch.int32, device=flag.device)
        check(lib().zepp_wait_geq(_p(flag), ctypes.c_uint64(value), int(limit_ms), _p(res), _stream()))
        return res


C = _C()
