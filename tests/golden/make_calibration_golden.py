"""Generate tests/golden/calibration_vectors.json from the reference's own calibration code.

Run in a container where OpenBitSys/BitDecoding-FP4 is mounted (see --reference):

    python tests/golden/make_calibration_golden.py [--reference <checkout of OpenBitSys/BitDecoding-FP4>]

It imports ``src/nvfp4_decode_kernel/reference.py`` (``online_probability_scale_statistics``) and
``src/nvfp4_vllm/probability_calibration.py`` (``threshold_for_code``,
``fit_probability_threshold``; pure Python), feeds them seeded inputs and stores inputs and
outputs. The scores are regenerated from the recorded seeds by the tests, so only the statistics
are stored.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import sys
from pathlib import Path

import torch


def seeded_scores(seed: int, heads: int, tokens: int) -> torch.Tensor:
    """Unscaled QK scores with a few dominant positions per head, as attention rows have."""
    gen = torch.Generator().manual_seed(seed)
    scores = 8.0 * torch.randn(heads, tokens, generator=gen)
    for h in range(heads):
        hot = torch.randperm(tokens, generator=gen)[:5]
        scores[h, hot] += 60.0 * torch.rand(5, generator=gen)
    return scores


CASES = [
    dict(seed=1, heads=4, tokens=700, fp4_tokens=640, sink_tokens=16, multiplier=1.0),
    dict(seed=2, heads=2, tokens=384, fp4_tokens=384, sink_tokens=4, multiplier=8.0),
    dict(seed=3, heads=8, tokens=1300, fp4_tokens=1280, sink_tokens=0, multiplier=8.0),
    dict(seed=4, heads=1, tokens=257, fp4_tokens=128, sink_tokens=16, multiplier=8.0),
]


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default="/root/reference")
    args = parser.parse_args()
    src = Path(args.reference) / "src"
    sys.path.insert(0, str(src))
    from nvfp4_decode_kernel.reference import online_probability_scale_statistics  # noqa: E402

    spec = importlib.util.spec_from_file_location("ref_probability_calibration",
                                                  src / "nvfp4_vllm" / "probability_calibration.py")
    calibration = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(calibration)

    out = {"statistics": [], "threshold_for_code": {}, "fits": []}
    samples_by_case = []
    for case in CASES:
        scores = seeded_scores(case["seed"], case["heads"], case["tokens"])
        stats = online_probability_scale_statistics(
            scores, fp4_tokens=case["fp4_tokens"], head_dim=128, sink_tokens=case["sink_tokens"],
            probability_multiplier=case["multiplier"])
        out["statistics"].append({
            "case": case, "group_count": stats["group_count"], "divisors": stats["divisors"],
            "by_code": {code: {"groups": b["groups"],
                               "winner_counts": [b["winner_counts"][str(d)] for d in stats["divisors"]],
                               "error_sum": [b["error_sum"][str(d)] for d in stats["divisors"]],
                               "oracle_error_sum": b["oracle_error_sum"]}
                        for code, b in stats["by_amax_e4m3_code"].items()},
        })
        samples_by_case.append(stats["by_amax_e4m3_code"])
    for code in range(-1, 126):
        out["threshold_for_code"][str(code)] = calibration.threshold_for_code(code)

    def sample(position, by_code):
        return {"position": position,
                "codes": {int(code): {"groups": b["groups"], "error_sum": dict(b["error_sum"])}
                          for code, b in by_code.items()}}

    # two workers, three query positions, multiplier 8: the statistics of cases 2-4 reused as samples
    workers = [
        [sample(128, samples_by_case[1]), sample(640, samples_by_case[2]), sample(1100, samples_by_case[3])],
        [sample(128, samples_by_case[2]), sample(640, samples_by_case[3]), sample(1100, samples_by_case[1])],
    ]
    out["fits"].append({"workers": workers, "multiplier": 8.0,
                        "report": calibration.fit_probability_threshold(workers, 8.0)})
    single = [[sample(200, samples_by_case[0]), sample(500, samples_by_case[1])]]
    out["fits"].append({"workers": single, "multiplier": 1.0,
                        "report": calibration.fit_probability_threshold(single, 1.0)})
    path = Path(__file__).parent / "calibration_vectors.json"
    path.write_text(json.dumps(out))
    print(f"wrote {path} ({path.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
