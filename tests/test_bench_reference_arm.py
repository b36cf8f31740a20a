"""The reference arm of the benchmark (`bench.py --impl reference`) runs on host cores only: its JSON line and what it
times.  No GPU."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [line for line in res.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["higher_is_better"] is True
    assert line["metric"] == "fused qnorm/RoPE/FP8-insert tokens/s" and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["value"] > 0 and line["gpu_launches"] == 0
    assert line["config"]["workload"] == "long_prefill"
    baseline = line["cpu_baseline"]
    # the upstream torch function itself wherever its test file can be read (a checkout, or the verified copy under
    # oracle/_ref); the restatement only where neither is present
    from oracle import ref_loader

    assert baseline["kind"] == ("reference" if ref_loader.hot_path_test_root() is not None else "port")
    assert baseline["cores"] >= 1 and baseline["value"] == line["value"] and "ref_impl" in baseline["sample"] or baseline["kind"] == "port"
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
