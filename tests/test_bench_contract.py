"""The benchmark's output contract: one JSON line with the agreed keys, for the CPU reference arm (runs anywhere)
and for the GPU arm (needs a B200)."""

import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT

BENCH = os.path.join(ROOT, "bench.py")
COMMON = ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
          "dtype", "data", "config", "e2e", "gpu_launches", "cpu_baseline")


def run_bench(*flags):
    res = subprocess.run([sys.executable, BENCH, *flags], capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [line for line in res.stdout.splitlines() if line.strip()]
    assert len(lines) == 1, "exactly one JSON line on stdout"
    return json.loads(lines[0])


def test_reference_arm_prints_the_contract_line():
    d = run_bench("--impl", "reference", "--steps", "1", "--warmup", "0")
    for key in COMMON:
        assert key in d, key
    assert d["impl"] == "reference" and d["metric"] == "gpt2_124m_fwd_tokens_per_s" and d["unit"] == "tokens/s"
    assert d["value"] > 0 and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"]


def test_reference_arm_under_torchrun_prints_once():
    """Launched as two ranks (the way the multi-GPU arm is launched), rank 0 alone runs the CPU arm and prints; the
    other rank exits 0 without output.  torchrun sets OMP_NUM_THREADS=1: the arm must still use the host's cores."""
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", "29577", BENCH, "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [line for line in res.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))


@pytest.mark.gpu
def test_gpu_arm_prints_the_contract_line():
    d = run_bench("--steps", "2", "--warmup", "3", "--skip-cpu-baseline")
    for key in COMMON + ("roofline", "clocks"):
        assert key in d, key
    assert d["n_gpus"] == 1 and d["steps"] == 2 and d["warmup"] == 3 and d["scaling"] == "strong" and d["dtype"] == "fp16"
    assert d["value"] > 1e6 and abs(d["value"] - 512 * 300 / (d["ms_per_step"] * 1e-3)) < 1.0
    # library kernels inside the timed region: embedding + 12 x (c_attn, attention, c_proj + statistics merge, c_fc,
    # c_proj + statistics merge; none after the last) + final LayerNorm + lm_head
    assert d["gpu_launches"] == 86 * 2 and d["device_status"] == 0
    e2e = d["e2e"]
    assert e2e["h2d_bytes_per_step"] == 512 * 300 * 8 and e2e["d2h_bytes_per_step"] == 512 * 300 * 8
    assert 0 < e2e["value"] and e2e["value"] != d["value"]
    r = d["roofline"]
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert 0.3 < r["frac"] < 1.2 and (r["traffic"] is None or r["traffic"] > 0.5 * r["traffic_algorithmic"]) and r["traffic_source"]
    assert d["ms_per_step_x_sm_mhz"] is None or d["ms_per_step_x_sm_mhz"] > 0
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
    assert "workload" in d["config"] and "l2" in d["config"]


@pytest.mark.gpu
def test_decode_mode_prints_one_line_with_an_hbm_roofline():
    """`bench.py --decode`: generation with the key/value cache (small batch, few tokens: a functional check of the
    mode; its own assertions require the replayed decode steps to regenerate the first pass's ids)."""
    d = run_bench("--decode", "--global-batch", "8", "--new-tokens", "6", "--steps", "3")
    assert d["metric"] == "gpt2_124m_decode_tokens_per_s" and d["unit"] == "tokens/s" and d["n_gpus"] == 1
    assert d["value"] > 0 and abs(d["value"] - 8 / (d["ms_per_decode_step"] * 1e-3)) < 1e-3 * d["value"]
    assert d["config"]["launches_per_decode_step"] == 88  # 1 + 12 x 7 - 1 + final LayerNorm + lm_head + reduce + append
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert r["algorithmic_bytes_per_step"] == r["weights_bytes"] + r["kv_cache_bytes"]
