"""The reference arm of bench.py runs on CPU and prints exactly one JSON line with the agreed keys."""

import json
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_json_line():
    res = subprocess.run(
        [sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1", "--cpu-rows", "16"],
        capture_output=True, text=True, timeout=300, cwd=str(REPO),
    )
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, f"expected one line on stdout, got {len(lines)}"
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    for key in ("metric", "value", "n_gpus", "steps", "warmup", "ms_per_step", "scaling", "vs_baseline", "dtype", "data", "config",
                "cpu_baseline", "e2e", "gpu_launches"):
        assert key in d, key
    assert d["vs_baseline"] is None and d["value"] > 0
    assert "workload" in d["config"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_flop_counts_match_the_stated_formulas():
    sys.path.insert(0, str(REPO))
    import bench

    s = bench.SHAPES
    assert abs(bench.algorithmic_flops("swiglu", s["swiglu"]) - 11.545e12) < 0.01e12
    assert abs(bench.algorithmic_flops("cross_entropy", s["cross_entropy"]) - 25.821e12) < 0.01e12
    assert abs(bench.algorithmic_flops("qknorm_rope", s["qknorm_rope"]) - 2.474e12) < 0.01e12
    assert abs(bench.algorithmic_flops("sigmoid", s["sigmoid"]) - 5.154e12) < 0.01e12
    assert abs(bench.algorithmic_flops("sigmoid_glu", s["sigmoid_glu"]) - 10.308e12) < 0.01e12
