"""GPU: bench.py prints one JSON line with the keys its consumers rely on, for the default workload and the skinny one."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("extra", [[], ["--workload", "skinny", "--m", "4"]])
def test_bench_line_has_the_contract_keys(cuda, extra):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "4", "--warmup", "3", "--no-cpu-baseline"] + extra,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "roofline", "e2e", "gpu_launches", "clocks"):
        assert k in line, k
    assert line["steps"] == 4 and line["n_gpus"] == 1 and line["value"] > 0 and line["dtype"] == "u8"
    assert "workload" in line["config"] and "model" not in line["config"]
    roof = line["roofline"]
    for k in ("bound", "achieved", "peak", "unit", "frac", "traffic"):
        assert k in roof, k
    assert roof["bound"] in ("hbm", "tensor") and abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-6
    e2e = line["e2e"]
    assert e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0 and 0 < e2e["value"] < line["value"]
    assert line["gpu_launches"] >= 2 * line["steps"]
    assert "sm_mhz" in line["clocks"] and "reasons" in line["clocks"]
    if not extra:
        # the default line carries the other parts of the metric as sections; a section that failed would hold "error"
        for name in ("skinny", "helpers", "mlp_mnist", "conv2d_q", "mlp_block_rows"):
            assert name in line and "error" not in line[name], (name, line.get(name))
        assert line["mlp_mnist"]["fused_output_equals_layer_by_layer"] is True
        assert line["mlp_mnist"]["batch_streams"]["outputs_equal_single_stream"] is True
        assert line["conv2d_q"]["channels_last_equals_nchw_result"] is True
        for k in ("get_min_max", "quantize_u8", "dynamic_quantize_rows", "dequantize"):
            assert line["helpers"][k]["frac_of_measured"] > 0
        assert e2e["frac_of_h2d_ceiling"] > 0 and e2e["h2d_ceiling_gbs"] > 0   # (no upper bound: the host side is shared)
