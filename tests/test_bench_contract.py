"""The bench's reference arm runs on the CPU (the reference's host loop on all
host cores), so its one-line JSON contract can be checked without a GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    run = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
         "--small", "--steps", "1", "--warmup", "1"],
        capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [l for l in run.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, run.stdout
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup",
                "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["unit"] == "Gitems/s" and line["higher_is_better"] is True
    assert line["vs_baseline"] is None and line["data"] == "synthetic"
    assert "workload" in line["config"]
    assert line["value"] > 0 and line["ms_per_step"] > 0
    base = line["cpu_baseline"]
    assert base["kind"] in ("port", "reference") and base["cores"] >= 1
    assert base["sample"] and base["value"] == line["value"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == line["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0
