"""The benchmark's one JSON line: keys and types that the harness around
bench.py reads, checked on the reduced workload so that it runs in seconds."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _line(*extra):
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--workload", "deep_brn_mlp_small",
                          "--steps", "3", "--warmup", "3", *extra], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    return json.loads(lines[0])


def test_bench_line_of_the_library():
    d = _line()
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks", "roofline", "cpu_baseline"):
        assert key in d, key
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["warmup"] >= 3 and d["higher_is_better"] is True
    assert d["scaling"] == "weak" and d["vs_baseline"] is None and d["data"] == "synthetic" and d["dtype"] == "f32"
    assert "workload" in d["config"] and "model" not in d["config"]
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["gpu_launches"] > 0
    e = d["e2e"]
    assert e["value"] > 0 and e["unit"] == d["unit"] and e["h2d_bytes_per_step"] > 0 and e["d2h_bytes_per_step"] > 0
    assert e["value"] != d["value"]
    r = d["roofline"]
    assert r["bound"] in ("hbm", "tensor") and r["unit"] in ("GB/s", "TFLOP/s")
    assert r["achieved"] > 0 and r["peak"] > 0 and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9 and "traffic" in r
    c = d["cpu_baseline"]
    assert c["value"] > 0 and c["cores"] >= 1 and c["kind"] in ("reference", "port") and c["sample"] and c["unit"] == d["unit"]
    assert set(d["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
    # The boundary as the reference calls it (row pointers in, a loss per step), the
    # range guard's counters, and the two records that only exist on several GPUs.
    dr = d["e2e_dropin"]
    assert dr["value"] > 0 and dr["unit"] == d["unit"] and dr["h2d_bytes_per_step"] == e["h2d_bytes_per_step"]
    assert e["in_order"]["value"] > 0
    assert d["range_guard"] == {"operand_tensors_flagged": 0, "products_on_fp32_fallback": 0, "tensors_split_again": 0,
                                "note": d["range_guard"]["note"]}
    assert d["comm"] is None and d["strong"] is None


def test_bench_line_of_the_reference_arm():
    d = _line("--impl", "reference", "--steps", "2", "--warmup", "1")
    assert d["impl"] == "reference" and d["value"] > 0 and d["metric"] and d["unit"]
    assert d["e2e"]["value"] == d["value"] and d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["cpu_baseline"]["value"] == d["value"] and d["cpu_baseline"]["kind"] in ("reference", "port")
