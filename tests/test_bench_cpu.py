"""The CPU arms of bench.py (the oracle timed as the baseline) run and report sane figures; no GPU."""

import importlib.util
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_cpu_samples_run():
    bench = _bench()
    for page_tokens in (64, 128):
        assert bench.cpu_sample_step(640, threads=2, page_tokens=page_tokens) > 0
    assert bench.mla_cpu_sample(256, heads=8, threads=2) > 0


def test_mla_reference_arm_prints_one_contract_line():
    run = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--workload", "mla", "--impl", "reference",
                          "--steps", "1", "--warmup", "3"], capture_output=True, text=True, timeout=600, check=True)
    lines = [line for line in run.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "mla_decode_attn_us_per_step"
    assert line["unit"] == "us/step" and line["higher_is_better"] is False and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
