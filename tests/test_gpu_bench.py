"""GPU: bench.py prints one JSON line with the agreed keys, for the per-call workload and for the
mask-caching trace (tiny shapes)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                         timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-3000:]
    return json.loads(out.stdout.strip().splitlines()[-1])


def test_call_workload_line():
    d = _run("--workload", "tiny", "--steps", "3", "--warmup", "3", "--cpu-blocks", "4")
    assert d["metric"] == "dfs_attn_effective_tflops" and d["unit"] == "TFLOP/s" and d["value"] > 0
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["warmup"] >= 3 and d["higher_is_better"] is True
    assert d["dtype"] == "bf16" and d["data"] == "synthetic" and d["config"]["workload"] == "tiny"
    assert d["gpu_launches"] > 0 and d["vs_baseline"] is None
    assert d["e2e"]["value"] > 0 and d["e2e"]["h2d_bytes_per_step"] > 0 and d["e2e"]["d2h_bytes_per_step"] > 0
    r = d["roofline"]
    assert r["bound"] == "tensor" and r["achieved"] > 0 and r["peak"] > 0 and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] > 0
    assert {"permute_ms", "score_select_ms", "attention_ms", "fused_prepare_ms"} <= set(d["stages"])
    assert "sm_mhz" in d["clocks"] and "reasons" in d["clocks"]
    assert d["stages"]["kp_attention_ms"] > 0 and 0 < d["stages"]["kp_tiles_kept_frac"] <= 1
    assert d["stages"]["dense_attention_ms"] > 0 and d["ms_x_mhz"] > 0
    e = d["e2e"]
    assert e["copy_only_ms"] > 0 and e["h2d_gbs_per_gpu"] > 0 and e["floor_ms"] >= e["copy_only_ms"]
    # the other configurations ride in the same line: five Wan calls and the 1-layer trace
    assert len(d["configs"]) == 6 and all(v.get("tflops", 0) > 0 for v in d["configs"].values()), d["configs"]


def test_wan_workload_line_times_the_guidance_pair():
    d = _run("--workload", "tiny_wan", "--steps", "3", "--warmup", "3", "--cpu-blocks", "4", "--no-extras")
    assert d["value"] > 0 and d["config"]["workload"] == "tiny_wan"
    assert d["stages"]["cfg_two_calls_ms"] > 0 and d["stages"]["cfg_pair_call_ms"] > 0


def test_trace_workload_line():
    d = _run("--workload", "tiny_trace", "--steps", "1", "--warmup", "1")
    assert d["value"] > 0 and d["config"]["denoising_steps"] == 50 and d["config"]["layers"] == 2
    calls = d["calls_ms"]
    # sparsity 0.5 with a decrement of 0.1: 12 dense steps, refreshes at steps 12 / 24 / 36 / 48, the
    # rest on cached lists -- per layer
    assert calls["dense"]["calls_per_trace"] == 24
    assert sum(v["calls_per_trace"] for k, v in calls.items() if k.startswith("refresh")) == 8
    assert sum(v["calls_per_trace"] for k, v in calls.items() if k.startswith("cached")) == 68
    # per call one status snapshot; dense: + attention; cached: + permute + attention; refresh: + four scoring kernels
    assert d["gpu_launches"] == 24 * 2 + 8 * 7 + 68 * 3 and d["ms_x_mhz"] > 0
