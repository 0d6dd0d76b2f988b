"""bench.py's reference arm on the host cores: the JSON line the driver parses (no GPU needed)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench(*args, env=None):
    e = dict(os.environ, **(env or {}))
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], env=e, capture_output=True, text=True,
                          timeout=600, cwd=ROOT)


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    r = _bench("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for k in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert k in d, k
    assert d["impl"] == "reference" and d["metric"] == "moe_layer_tflops" and d["unit"] == "TFLOP/s"
    assert d["value"] > 0 and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"]


def test_reference_arm_is_silent_on_other_ranks():
    r = _bench("--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1",
               env={"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert r.returncode == 0, r.stderr[-2000:]
    assert not [ln for ln in r.stdout.splitlines() if ln.startswith("{")]


def test_layer_roofline_terms_on_a_hand_computed_routing():
    """The roofline the bench line reports, evaluated by hand on a two-rank routing: FLOPs 6·H·I·rows, NVLink
    2·H·(max(out, in) dispatch rows + max(out, in) combine rows) at 900 GB/s per direction, HBM 6·H·I per touched expert."""
    import importlib.util
    from types import SimpleNamespace

    import torch
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    shape = SimpleNamespace(hidden=1024, ffn_hidden=512)
    W, gpe = 2, 3
    # sps[s, d*gpe + j]: copies of source s on group j of rank d
    sps = torch.tensor([[4, 0, 2, 1, 0, 0],
                        [0, 3, 0, 0, 5, 2]])
    uc = torch.tensor([[5, 1], [3, 6]])                  # tokens of s with a copy on d
    splits = sps.sum(0)                                  # rows per (rank, group): [4, 3, 2 | 1, 5, 2]
    r = bench.layer_roofline(shape, W, gpe, sps, uc, splits, hbm_gbs=5000.0, bf16_tf=1000.0)
    H, I = 1024, 512
    rows = [4 + 3 + 2, 1 + 5 + 2]
    assert r["rows_max"] == 9 and r["rows_min"] == 8
    assert abs(r["t_flop_us"] - 6 * H * I * 9 / 1e15 * 1e6) < 1e-9
    # dispatch: rank 0 sends 1 token row and receives 3; combine: owner 0 returns 3 rows to rank 1 and gets 1 back
    assert r["dispatch_rows_out_in_max"] == [3, 3] and r["combine_rows_out_in_max"] == [3, 3]
    assert abs(r["t_nvlink_us"] - 2 * H * (3 + 3) / 900e9 * 1e6) < 1e-9
    assert abs(r["t_hbm_weights_us"] - 6 * H * I * 3 / 5000e9 * 1e6) < 1e-9
    assert r["t_roof_3term_us"] >= r["t_roof_2term_us"] >= max(r["t_flop_us"], r["t_nvlink_us"]) - 1e-12
    assert rows[0] == int(splits[:3].sum())
