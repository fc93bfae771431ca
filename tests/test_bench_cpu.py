"""The reference arm of the benchmark needs no GPU: run it here on a short sample and check the line it prints
(the reference's C dequantiser from oracle/_ref + fp32 matmul on the host cores, same metric, unit and config as the
GPU arm).  Skipped where oracle/_ref has not been built (it is built from the reference tree, which only this
container holds)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.timeout(300)
def test_reference_arm_prints_the_contract_line(oracle):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                        "--cpu-seconds", "1"], capture_output=True, text=True, timeout=280, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    if "unavailable" in line:
        pytest.skip(line["unavailable"])
    assert line["impl"] == "reference" and line["metric"] == "moe_layer_tokens_per_s" and line["unit"] == "token-layers/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["value"] > 0
    assert line["config"]["workload"].startswith("decode stack") and "model" not in line["config"]
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0
