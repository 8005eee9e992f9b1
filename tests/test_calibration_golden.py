"""Calibration producers against vectors produced by the reference's own code
(tests/golden/make_calibration_golden.py): the threshold fit (host logic of the plugin) and the CPU
oracle of the probability-scale statistic."""

import json
import math
from pathlib import Path

import pytest
import torch

from oracle import calibration_oracle

GOLDEN = json.loads((Path(__file__).parent / "golden" / "calibration_vectors.json").read_text())


def seeded_scores(seed, heads, tokens):
    """The generator of tests/golden/make_calibration_golden.py."""
    gen = torch.Generator().manual_seed(seed)
    scores = 8.0 * torch.randn(heads, tokens, generator=gen)
    for h in range(heads):
        hot = torch.randperm(tokens, generator=gen)[:5]
        scores[h, hot] += 60.0 * torch.rand(5, generator=gen)
    return scores


def test_threshold_for_code_matches_reference():
    from nvfp4_vllm.probability_calibration import threshold_for_code

    for code, want in GOLDEN["threshold_for_code"].items():
        assert threshold_for_code(int(code)) == want, code
    with pytest.raises(ValueError):
        threshold_for_code(126)


def _int_codes(workers):
    return [[{"position": s["position"], "codes": {int(c): b for c, b in s["codes"].items()}} for s in worker]
            for worker in workers]


@pytest.mark.parametrize("index", range(len(GOLDEN["fits"])))
def test_fit_probability_threshold_matches_reference(index):
    from nvfp4_vllm.probability_calibration import fit_probability_threshold

    case = GOLDEN["fits"][index]
    got = fit_probability_threshold(_int_codes(case["workers"]), case["multiplier"])
    want = case["report"]
    assert got["tau"] == want["tau"] and got["threshold_code"] == want["threshold_code"]
    assert got["samples"] == want["samples"] and got["groups"] == want["groups"]
    assert got["squared_error"] == want["squared_error"]
    assert got["amax6_squared_error"] == want["amax6_squared_error"]
    assert got["folds"] == want["folds"]
    assert {k: got[k] for k in ("c", "rule", "validation", "source")} == {k: want[k] for k in ("c", "rule", "validation", "source")}


def test_fit_rejects_bad_input():
    from nvfp4_vllm.probability_calibration import ProbabilityCalibration, fit_probability_threshold

    one_position = [[{"position": 5, "codes": {3: {"groups": 1, "error_sum": {"2": 0.1, "6": 0.2}}}}]]
    with pytest.raises(ValueError):
        fit_probability_threshold(one_position, 8.0)
    with pytest.raises(ValueError):
        fit_probability_threshold(one_position * 2, 0.0)
    with pytest.raises(ValueError):
        ProbabilityCalibration(200, 8.0)
    collector = ProbabilityCalibration(1024, 8.0, samples=4)
    assert collector.positions == [128, 426, 724, 1023]


@pytest.mark.parametrize("index", range(len(GOLDEN["statistics"])))
def test_statistic_oracle_matches_reference(index):
    entry = GOLDEN["statistics"][index]
    case = entry["case"]
    scores = seeded_scores(case["seed"], case["heads"], case["tokens"])
    got = calibration_oracle.probability_scale_statistics(
        scores, fp4_tokens=case["fp4_tokens"], head_dim=128, sink_tokens=case["sink_tokens"],
        probability_multiplier=case["multiplier"])
    want = {int(code): bucket for code, bucket in entry["by_code"].items()}
    assert entry["divisors"] == [6, 4, 3, 2]
    assert set(got) == set(want)
    assert sum(b["groups"] for b in got.values()) == entry["group_count"]
    for code, bucket in want.items():
        assert got[code]["groups"] == bucket["groups"]
        assert got[code]["winner_counts"] == bucket["winner_counts"]
        for a, b in zip(got[code]["error_sum"], bucket["error_sum"]):
            assert math.isclose(a, b, rel_tol=1e-12, abs_tol=1e-30)
        assert math.isclose(got[code]["oracle_error_sum"], bucket["oracle_error_sum"], rel_tol=1e-12, abs_tol=1e-30)
