"""zepp_routed_meta_noalloc through the C ABI against zepp_routed_meta.

The no-alloc variant exists for hosts that cannot allocate device memory at planning time (the GPU
already belongs to their own memory pool, or the planning thread must never block in the
allocator): it takes no workspace and uses a fixed 1 MiB scratch array inside the library.  Both
entry points run the same kernels, so every output must be identical, including on a second call
that finds the first call's leftovers in the shared scratch.  This file sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import planner as op
from zepp_b200._ext import check, lib

pytestmark = pytest.mark.gpu
NAMES = ("vce", "splits", "scatter_index", "sps", "uc", "demands", "dplan", "cplan")


def _buffers(R, L, S, K, gpe, dev):
    NN, E = R // L, R * gpe
    return dict(vce=torch.full((R * S * K,), -3, dtype=torch.int32, device=dev),
                splits=torch.full((E,), -3, dtype=torch.int32, device=dev),
                scatter_index=torch.full((R * S * K,), -3, dtype=torch.int32, device=dev),
                sps=torch.full((R * E,), -3, dtype=torch.int32, device=dev),
                uc=torch.full((R * (R + NN),), -3, dtype=torch.int32, device=dev),
                demands=torch.full((8,), -3, dtype=torch.int64, device=dev),
                dplan=torch.zeros(lib().zepp_dispatch_plan_words(L, NN), dtype=torch.int64, device=dev),
                cplan=torch.zeros(4 * R + 2, dtype=torch.int64, device=dev))


def _call(noalloc, vce_in, R, L, S, K, gpe, rank):
    dev = vce_in.device
    o = _buffers(R, L, S, K, gpe, dev)
    caps = (ctypes.c_int64 * 8)(*([1 << 40] * 8))
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    head = (ctypes.c_void_p(0), p(vce_in), R, L, S, K, gpe - 1, gpe, rank, 0, 2, caps, S * K, p(o["vce"]),
            ctypes.c_void_p(0), p(o["splits"]), p(o["scatter_index"]), p(o["sps"]), p(o["uc"]), p(o["demands"]),
            p(o["dplan"]), p(o["cplan"]) if R == L else ctypes.c_void_p(0))
    if noalloc:
        check(lib().zepp_routed_meta_noalloc(*head, stream))
    else:
        ws = torch.full((lib().zepp_meta_workspace_bytes(R, S, K, gpe),), 0x5A, dtype=torch.uint8, device=dev)
        check(lib().zepp_routed_meta(*head, p(ws), stream))
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in o.items()}


def test_noalloc_matches_workspace_variant_twice_in_a_row():
    rng = np.random.default_rng(7)
    # second case smaller and differently shaped than the first: it runs on the first call's leftovers
    for (R, L, S, K, gpe) in ((8, 8, 136, 8, 11), (4, 2, 24, 6, 5)):
        vce_in = torch.from_numpy(rng.integers(0, R * gpe, size=R * S * K, dtype=np.int32)).cuda()
        for rank in (0, R - 1):
            ref = _call(False, vce_in, R, L, S, K, gpe, rank)
            got = _call(True, vce_in, R, L, S, K, gpe, rank)
            for name in NAMES:
                assert np.array_equal(got[name], ref[name]), (R, L, S, K, gpe, rank, name)
            assert int(ref["splits"].sum()) == R * S * K and ref["demands"][7] == 0
        # and against the CPU oracle directly, so this file stands on its own
        splits, scat, sps, uc = op.routed_meta(vce_in.cpu().numpy().reshape(R * S, K), R, S, gpe, R // L, L)
        assert np.array_equal(got["splits"], splits) and np.array_equal(got["scatter_index"], scat.reshape(-1))
        assert np.array_equal(got["sps"], sps.reshape(-1)) and np.array_equal(got["uc"], uc.reshape(-1))
        assert got["demands"][:7].tolist() == op.demands_from_meta(sps, uc, R, L, gpe)


def test_noalloc_refuses_routings_beyond_its_scratch():
    R, L, S, K, gpe = 64, 4, 1024, 8, 23           # needs about 3 MiB, well over the 1 MiB built-in scratch
    assert lib().zepp_meta_workspace_bytes(R, S, K, gpe) > (1 << 20)
    vce_in = torch.zeros(8, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="built-in scratch holds"):
        _call(True, vce_in, R, L, S, K, gpe, 0)
    assert float(torch.ones(2, device="cuda").sum()) == 2.0
