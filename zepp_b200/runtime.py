"""Python handles of the C-ABI runtime objects (symmetric arena per rank, layer)."""
import ctypes

import numpy as np
import torch

from . import constants
from ._ext import LayerCfg, check, lib

TABLES = {"loads": (0, torch.int32), "phys_own": (1, torch.int32), "vce": (2, torch.int32),
          "probs_all": (3, torch.float32), "splits": (4, torch.int32), "scatter_index": (5, torch.int32),
          "sps": (6, torch.int32), "uc": (7, torch.int32), "demands": (8, torch.int64), "dplan": (9, torch.int64),
          "cplan": (10, torch.int64), "route_ws": (11, torch.int32), "swap_block": (12, torch.int64),
          "m_this": (13, torch.int32), "row_tok": (14, torch.int32), "act": (15, torch.bfloat16),
          "recv": (16, torch.bfloat16), "p2l": (17, torch.int32), "l2p": (18, torch.int32),
          "n_tiles": (19, torch.int32), "panel": (20, torch.bfloat16), "gate": (21, torch.int64),
          "sched": (22, torch.int32)}


def make_cfg(cfg, caps, c_num, c_den):
    s = cfg.shape
    c = LayerCfg()
    c.num_experts, c.topk, c.hidden, c.ffn_hidden = s.num_experts, s.topk, s.hidden, s.ffn_hidden
    c.act = 1 if s.act == "swiglu" else 0
    c.ranks, c.ranks_per_node, c.max_tokens_per_rank = cfg.ranks, cfg.ranks_per_node, cfg.max_tokens_per_rank
    c.strategy = 0 if cfg.comm_strategy == "overlap" else 1
    c.swap, c.redundant_slots_per_rank = int(cfg.swap), cfg.redundant_slots_per_rank
    c.sm_margin, c.gpu_plan = cfg.sm_margin, int(cfg.gpu_plan)
    c.c_num, c.c_den = c_num, c_den
    for i, v in enumerate(caps.as_list()):
        c.caps[i] = int(v)
    return c


def gather_blobs(group, blob: bytes) -> bytes:
    """All-gather one fixed-size byte string per rank over a torch.distributed group (any backend);
    returns the concatenation in rank order.  This is the only use of the process group besides
    barriers: the bootstrap of the symmetric arenas."""
    import torch.distributed as dist
    world = dist.get_world_size(group=group)
    out = [None] * world
    dist.all_gather_object(out, blob, group=group)
    assert all(isinstance(b, bytes) and len(b) == len(blob) for b in out)
    return b"".join(out)


class Runtime:
    """One rank's symmetric arena.  `create_group` maps the arenas of all ranks into each other:
    over CUDA IPC handles exchanged through a torch.distributed group (one process per GPU), or by
    plain pointers when several ranks live in this process on one GPU."""

    def __init__(self, rank, world, device_index, arena_bytes):
        self.h = ctypes.c_void_p()
        self.rank, self.world = rank, world
        check(lib().zepp_rt_create(rank, world, device_index, ctypes.c_size_t(arena_bytes), ctypes.byref(self.h)))
        check(lib().zepp_rt_set_wait_limit_ms(self.h, constants.WAIT_LIMIT_MS))

    def set_wait_limit_ms(self, ms):
        check(lib().zepp_rt_set_wait_limit_ms(self.h, int(ms)))

    @property
    def sm_count(self):
        return lib().zepp_rt_sm_count(self.h)

    def exchange_handles(self, group):
        """Collective over `group`: all-gather the 64-byte IPC handles and map every peer's arena."""
        import torch.distributed as dist
        blob = (ctypes.c_uint8 * 64)()
        check(lib().zepp_rt_ipc_handle(self.h, blob))
        raw = gather_blobs(group, bytes(blob))
        check(lib().zepp_rt_open_peers(self.h, raw, self.world))
        dist.barrier(group=group)

    @staticmethod
    def link_local(rts):
        arr = (ctypes.c_void_p * len(rts))(*[r.h for r in rts])
        check(lib().zepp_rt_link_local(arr, len(rts)))

    def destroy(self):
        if self.h:
            lib().zepp_rt_destroy(self.h)
            self.h = ctypes.c_void_p()


class LayerHandle:
    def __init__(self, rt, ccfg):
        self.rt = rt
        self.h = ctypes.c_void_p()
        self.ccfg = ccfg
        check(lib().zepp_layer_create(rt.h, ctypes.byref(ccfg), ctypes.byref(self.h)))

    @staticmethod
    def arena_bytes(ccfg):
        return int(lib().zepp_layer_arena_bytes(ctypes.byref(ccfg)))

    def set_placement(self, pl):
        p2l = np.ascontiguousarray(pl.p2l.cpu().numpy().astype(np.int32))
        l2p = np.ascontiguousarray(pl.l2p.cpu().numpy().astype(np.int32))
        lc = np.ascontiguousarray(pl.lcnts.cpu().numpy().astype(np.int32))
        check(lib().zepp_layer_set_placement(self.h, p2l.ctypes.data_as(ctypes.c_void_p),
                                             l2p.ctypes.data_as(ctypes.c_void_p), lc.ctypes.data_as(ctypes.c_void_p),
                                             self._stream()))

    def set_tokens(self, tokens):
        check(lib().zepp_layer_set_tokens(self.h, int(tokens)))

    @staticmethod
    def _stream():
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def set_weights(self, w1, w2):
        assert w1.is_cuda and w2.is_cuda and w1.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16
        assert w1.is_contiguous() and w2.is_contiguous()
        check(lib().zepp_layer_set_weights(self.h, ctypes.c_void_p(w1.data_ptr()), ctypes.c_void_p(w2.data_ptr())))

    def weight_slots(self, gpe, ffn1, H, ffn):
        """The layer-owned weight slots (swap on) as tensors w1 [gpe, ffn1, H], w2 [gpe, H, ffn]."""
        p1, p2 = ctypes.c_void_p(), ctypes.c_void_p()
        check(lib().zepp_layer_weight_slots(self.h, ctypes.byref(p1), ctypes.byref(p2)))
        w1 = torch.as_tensor(_DevMem(p1.value, gpe * ffn1 * H, torch.bfloat16), device="cuda").view(torch.bfloat16)
        w2 = torch.as_tensor(_DevMem(p2.value, gpe * H * ffn, torch.bfloat16), device="cuda").view(torch.bfloat16)
        return w1.view(gpe, ffn1, H), w2.view(gpe, H, ffn)

    def prepare(self, ids, wts, phase=None):
        assert ids.is_cuda and ids.dtype == torch.int32 and ids.is_contiguous()
        assert wts.is_cuda and wts.dtype == torch.float32 and wts.is_contiguous()
        a = (self.h, ctypes.c_void_p(ids.data_ptr()), ctypes.c_void_p(wts.data_ptr()), self._stream())
        if phase is None:
            check(lib().zepp_layer_prepare(*a))
        else:
            check(lib().zepp_layer_prepare_phase(a[0], int(phase), *a[1:]))

    def forward(self, x, y, phase=None):
        assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
        a = (self.h, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()), self._stream())
        if phase is None:
            check(lib().zepp_layer_forward(*a))
        else:
            check(lib().zepp_layer_forward_phase(a[0], int(phase), *a[1:]))

    def step(self, ids, wts, x, y):
        check(lib().zepp_layer_step(self.h, ctypes.c_void_p(ids.data_ptr()), ctypes.c_void_p(wts.data_ptr()),
                                    ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()), self._stream()))

    def status(self):
        out = (ctypes.c_uint64 * 8)()
        check(lib().zepp_layer_status(self.h, self._stream(), out))
        return [int(v) for v in out]

    def trace(self):
        out = (ctypes.c_uint64 * 64)()
        check(lib().zepp_layer_trace(self.h, self._stream(), out))
        return [int(v) for v in out]

    def launches(self):
        v = ctypes.c_int64()
        check(lib().zepp_layer_gpu_launches(self.h, ctypes.byref(v)))
        return int(v.value)

    def table(self, name):
        """A planner product of the last prepare as a device tensor (a view of runtime memory)."""
        which, dtype = TABLES[name]
        p, n = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().zepp_layer_table(self.h, which, ctypes.byref(p), ctypes.byref(n)))
        item = torch.empty(0, dtype=dtype).element_size()
        holder = _DevMem(p.value, n.value // item, dtype)
        t = torch.as_tensor(holder, device="cuda")
        # the array interface cannot name bfloat16: it travels as int16 and is viewed back
        return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t

    def destroy(self):
        if self.h:
            lib().zepp_layer_destroy(self.h)
            self.h = ctypes.c_void_p()


class _DevMem:
    """Exposes a raw device range through __cuda_array_interface__."""
    _TYPESTR = {torch.int32: "<i4", torch.int64: "<i8", torch.float32: "<f4", torch.bfloat16: "<i2",
                torch.uint8: "|u1"}

    def __init__(self, ptr, count, dtype):
        self.dtype = dtype
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": self._TYPESTR[dtype], "data": (ptr, False),
                                         "version": 2}
