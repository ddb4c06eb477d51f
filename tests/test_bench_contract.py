"""What the benchmark script answers without a GPU: more than one GPU is refused with one line
and exit code 2, and the reference arm says in one JSON line why it is unavailable."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          cwd=ROOT, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line():
    p = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    lines = [ln for ln in (p.stdout + p.stderr).splitlines() if ln.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    p = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and "\n" not in rec["unavailable"]


def test_bytes_and_flops_the_roofline_fractions_rest_on():
    """The step's bytes and the prompt's flops for the benchmark's sizes, against the figures worked
    out by hand: 1,235,814,400 parameters at 2 bytes, 32,768 bytes of cache a token, and the products of
    a 2,048-token prompt with the last layer's feed-forward and the output matrix for one row only."""
    sys.path.insert(0, ROOT)
    import bench
    weight_bytes, kv_per_token, flops = bench.model_numbers(bench.LLAMA_1B)
    assert weight_bytes == 2 * 1_235_814_400
    assert kv_per_token == 2 * 16 * 8 * 64 * 2
    H, I, L, V, T = 2048, 8192, 16, 128256, 2048
    linear = 2 * T * L * (H * 3072 + H * H) + 2 * (T * (L - 1) + 1) * 3 * H * I
    attention = L * 4 * 32 * 64 * T * (T + 1) // 2
    assert flops(T) == linear + attention + 2 * V * H
    assert abs(flops(T) / 1e12 - 4.055) < 0.001
    w8, kv8, _ = bench.model_numbers(bench.LLAMA_8B)
    assert kv8 == 131072 and abs(w8 / 1e9 - 15.009) < 0.06      # the 8B model: layers, output matrix and norms (no token table)


import pytest


@pytest.mark.gpu
def test_the_benchmark_line_on_a_gpu():
    """One short run of the benchmark itself: one JSON line with the keys the contract names, launches
    counted, both timings of the step, and fractions that are fractions."""
    p = run("--steps", "8", "--warmup", "3", "--no-points")
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "ms_per_step_median", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks", "prefill", "roofline",
                "points", "dominant_kernel"):
        assert key in rec, key
    assert rec["n_gpus"] == 1 and rec["steps"] == 8 and rec["dtype"] == "bf16" and rec["higher_is_better"] is True
    assert len(rec["config"]) <= 20 and all(not isinstance(v, (dict, list)) for v in rec["config"].values())
    assert rec["config"]["layers"] == rec["config"]["layers_full"] == 16 and rec["config"]["global_batch"] == 8
    assert rec["gpu_launches"] >= 8 * 100
    assert abs(rec["value"] - 8 * 1000.0 / rec["ms_per_step"]) < 1.0
    assert 0 < rec["e2e"]["value"] <= rec["value"] * 1.05 and rec["e2e"]["h2d_bytes_per_step"] > 0 and rec["e2e"]["d2h_bytes_per_step"] > 0
    assert 0.2 < rec["roofline"]["frac"] < 1.1 and 0.2 < rec["prefill"]["frac"] < 1.1 and rec["prefill"]["tokens"] == 2048
    assert 0.2 < rec["dominant_kernel"]["frac"] < 1.1
