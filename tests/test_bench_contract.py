"""bench.py prints one JSON line with the keys its contract names (small scales so that it is quick)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, r.stdout
    return json.loads(lines[0])


def test_host_arm_line():
    out = _run("--impl", "reference", "--steps", "1", "--warmup", "1", "--scale", "12")
    assert out["impl"] == "reference" and out["unit"] == "GFLOP/s" and out["higher_is_better"] is True
    assert out["cpu_baseline"]["kind"] == "port" and out["cpu_baseline"]["cores"] >= 1
    assert out["cpu_baseline"]["value"] == out["value"] == out["e2e"]["value"]
    assert out["e2e"]["h2d_bytes_per_step"] == 0 and out["e2e"]["d2h_bytes_per_step"] == 0
    assert "sample" in out["cpu_baseline"]


@pytest.mark.gpu
def test_default_arm_line_on_a_small_graph(cuda):
    out = _run("--steps", "5", "--warmup", "3", "--scale", "15", "--e2e-steps", "1", "--c5-scale", "14", "--c5-degree", "16", "--c5-steps", "3")
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "roofline", "e2e", "gpu_launches", "clocks", "cpu_baseline"):
        assert key in out, key
    assert out["n_gpus"] == 1 and out["steps"] == 5 and out["vs_baseline"] is None and out["data"] == "synthetic"
    assert out["roofline"]["bound"] == "hbm" and out["roofline"]["achieved"] > 0 and out["roofline"]["peak"] > 0
    assert abs(out["roofline"]["frac"] - out["roofline"]["achieved"] / out["roofline"]["peak"]) < 1e-3
    assert out["e2e"]["h2d_bytes_per_step"] > 0 and out["e2e"]["d2h_bytes_per_step"] > 0 and out["e2e"]["value"] < out["value"]
    assert out["gpu_launches"] >= 5 and "workload" in out["config"]
    assert out["cpu_baseline"]["kind"] == "port" and out["cpu_baseline"]["value"] > 0
    # the line looks at what it timed, and carries bounds that are fractions of a peak
    assert out["check"]["ok"] is True and out["check"]["rows"] >= 4000 and out["check"]["max_scaled_err"] <= 1.0
    assert out["e2e"]["check"]["ok"] is True
    sc = out["e2e"]["scaled_call"]   # the same product through mps_spmm_host_scaled: fewer bytes up, same C
    assert sc["check_ok"] is True and sc["h2d_bytes_per_step"] < out["e2e"]["h2d_bytes_per_step"]
    r = out["roofline"]
    assert 0 < r["compulsory_frac"] < 1.5 and r["l2_peak_gbs"] > r["hbm_gather_gbs"] > 0 and 0 < r["l2_frac"] < 1.5
    assert r["nearest_bound"] in ("hbm_compulsory", "l2_gather", "hbm_measured_traffic", "own_stream_gather")
    assert 0 < r["stream_frac"] < 1.5 and r["stream_gather_gbs"] > 0
    c5 = out["c5_strong"]
    assert c5["scaling"] == "strong" and c5["check"]["ok"] is True and c5["ms_per_step"] > 0 and c5["n_gpus"] == 1
    assert set(c5["dim_sweep"]) == {"16", "64", "128"} and all(v["check_ok"] and v["ms_per_step"] > 0 for v in c5["dim_sweep"].values())
    assert out["reference_gpu"].get("best", {}).get("cost") in (8, 32) or "unavailable" in out["reference_gpu"]


@pytest.mark.gpu
def test_profiling_flags_slab_and_walk(cuda):
    """--slab R/N: one rank's share of an N-GPU weak-scaling run alone on this GPU; --walk 1: a warp per unit."""
    out = _run("--steps", "3", "--warmup", "3", "--scale", "14", "--dim", "16", "--slab", "1/2", "--walk", "1", "--no-c5", "--skip-baselines",
               "--no-probe", "--e2e-steps", "1")
    assert out["config"]["workload"].endswith("_slab1of2") and out["config"]["nodes"] == 1 << 15
    assert out["config"]["groups_per_unit"] == 8 and out["check"]["ok"] is True and out["e2e"]["check"]["ok"] is True
    assert "c5_strong" not in out and "cpu_baseline" not in out and "l2_frac" not in out["roofline"]
