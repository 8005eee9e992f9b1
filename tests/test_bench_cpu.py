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
    from oracle import cpu_arm

    bench = _bench()
    for page_tokens in (64, 128):
        assert cpu_arm.port_step_seconds(640, page_tokens=page_tokens) > 0
    seconds, kind = cpu_arm.step_seconds(640, heads_kv=2, ratio=4)
    assert seconds > 0 and kind in ("reference", "port")
    assert bench.mla_cpu_sample(256, heads=8, threads=2) > 0


def test_reference_arm_runs_the_small_workload_whole_and_prints_the_gpu_arms_config():
    """`--impl reference --workload cfg1` runs every row of the batch (no extrapolation) and prints one
    contract line whose `config` is the one the GPU arm prints for the same arguments, key for key."""
    run = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--workload", "cfg1", "--impl", "reference",
                          "--steps", "1", "--warmup", "3"], capture_output=True, text=True, timeout=600, check=True)
    lines = [line for line in run.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "decode_attn_us_per_step" and line["value"] > 0
    assert line["cpu_baseline"]["extrapolated_x"] == 1.0 and "every row whole" in line["cpu_baseline"]["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "us/step", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    bench = _bench()
    args = type("Args", (), dict(workload="cfg1", page_tokens=64, heads_q=0, heads_kv=0, batch=0, context=65536))()
    spec = bench.workload_spec(args)
    part = bench.partition(spec, 1, 0)
    assert line["config"] == bench.common_config(spec, part["text"], 64)


def test_partition_of_heads_then_rows():
    """KV-head groups first, then batch shards; a ragged batch is dealt longest-first in a snake."""
    bench = _bench()
    spec = dict(heads_q=32, heads_kv=4, lengths=[131072] * 32)
    for world, want in ((1, (4, 32)), (2, (2, 32)), (4, (1, 32)), (8, (1, 16))):
        shares = [bench.partition(spec, world, rank) for rank in range(world)]
        assert all((p["heads_kv"], len(p["lengths"])) == want for p in shares)
        assert sum(p["heads_kv"] * len(p["lengths"]) for p in shares) == 4 * 32
    ragged = dict(heads_q=32, heads_kv=8, lengths=bench.zipf_lengths(256, 1024, 131072, 1.2, seed=5))
    assert min(ragged["lengths"]) >= 1024 and max(ragged["lengths"]) <= 131072
    halves = [bench.partition(ragged, 8, rank, kv_groups=4) for rank in (0, 4)]
    tokens = [sum(p["lengths"]) for p in halves]
    assert sum(len(p["lengths"]) for p in halves) == 256 and abs(tokens[0] - tokens[1]) < 0.05 * sum(tokens)


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
