"""Calibration producers on the GPU: the FP64 key sums, the probability-scale statistic kernel
against the CPU oracle (itself pinned to the reference by test_calibration_golden.py), and the
runtime's measure -> mean -> active-shift path."""

import math

import pytest
import torch

from oracle import calibration_oracle
from test_calibration_golden import GOLDEN, seeded_scores

pytestmark = pytest.mark.gpu


def test_key_channel_sums():
    import bdfp4

    gen = torch.Generator().manual_seed(3)
    for tokens, heads in ((1, 2), (63, 1), (5000, 8), (70001, 4)):
        key = (torch.randn(tokens, heads, 128, generator=gen) * 3 + 0.5).to(torch.bfloat16).cuda()
        sums = torch.full((heads, 128), 1.5, dtype=torch.float64, device="cuda")  # accumulates
        bdfp4.key_channel_sums(key, sums, bdfp4.current_stream(key.device))
        want = key.double().sum(dim=0) + 1.5
        assert torch.allclose(sums, want, rtol=1e-13, atol=1e-9), (tokens, heads)
    # a strided source: tokens of a wider row
    wide = torch.randn(300, 3 * 4 * 128, generator=gen).to(torch.bfloat16).cuda()
    key = wide[:, 512:1024].view(300, 4, 128)
    sums = torch.zeros(4, 128, dtype=torch.float64, device="cuda")
    bdfp4.key_channel_sums(key, sums, bdfp4.current_stream(key.device))
    assert torch.allclose(sums, key.double().sum(dim=0), rtol=1e-13, atol=1e-9)


@pytest.mark.parametrize("index", range(len(GOLDEN["statistics"])))
def test_probability_statistics_match_oracle(index):
    """expf on the GPU and torch.exp on the CPU differ in the last bit, so a group whose maximum
    sits on an E4M3 rounding boundary may change bucket: counts are compared in total and per
    code within a small slack, error sums per divisor to 1e-4 relative."""
    from nvfp4_decode_kernel.reference import online_probability_scale_statistics

    case = GOLDEN["statistics"][index]["case"]
    scores = seeded_scores(case["seed"], case["heads"], case["tokens"])
    got = online_probability_scale_statistics(
        scores.cuda(), fp4_tokens=case["fp4_tokens"], head_dim=128, sink_tokens=case["sink_tokens"],
        probability_multiplier=case["multiplier"])
    want = calibration_oracle.probability_scale_statistics(
        scores, fp4_tokens=case["fp4_tokens"], head_dim=128, sink_tokens=case["sink_tokens"],
        probability_multiplier=case["multiplier"])
    groups = case["heads"] * case["fp4_tokens"] // 16
    assert got["group_count"] == groups == sum(b["groups"] for b in want.values())
    assert got["divisors"] == [6, 4, 3, 2]
    got_codes = {int(code): bucket for code, bucket in got["by_amax_e4m3_code"].items()}
    moved = sum(abs(got_codes.get(code, {"groups": 0})["groups"] - want.get(code, {"groups": 0})["groups"])
                for code in set(got_codes) | set(want))
    assert moved <= max(2, groups // 500), moved
    for i, divisor in enumerate(("6", "4", "3", "2")):
        total = math.fsum(b["error_sum"][i] for b in want.values())
        assert math.isclose(got["error_sum"][divisor], total, rel_tol=1e-4), divisor
        assert got["winner_counts"][divisor] == pytest.approx(sum(b["winner_counts"][i] for b in want.values()),
                                                               abs=max(2, groups // 500))
    assert math.isclose(got["oracle_error_sum"], math.fsum(b["oracle_error_sum"] for b in want.values()), rel_tol=1e-4)


def test_fitted_threshold_from_gpu_statistics_equals_the_oracle_fit():
    from nvfp4_decode_kernel.reference import online_probability_scale_statistics
    from nvfp4_vllm.probability_calibration import fit_probability_threshold

    def samples(statistic):
        out = []
        for position, seed in ((300, 11), (900, 12), (1500, 13)):
            scores = seeded_scores(seed, 8, position + 1)
            fp4 = (position // 128) * 128
            by_code = statistic(scores, fp4)
            out.append({"position": position, "codes": {
                int(code): {"groups": b["groups"], "error_sum": b["error_sum"]} for code, b in by_code.items()}})
        return [out]

    def on_gpu(scores, fp4):
        stats = online_probability_scale_statistics(scores.cuda(), fp4_tokens=fp4, head_dim=128,
                                                    probability_multiplier=8.0)
        return stats["by_amax_e4m3_code"]

    def on_cpu(scores, fp4):
        stats = calibration_oracle.probability_scale_statistics(scores, fp4_tokens=fp4, head_dim=128,
                                                                probability_multiplier=8.0)
        return {code: {"groups": b["groups"], "error_sum": {"6": b["error_sum"][0], "2": b["error_sum"][3]}}
                for code, b in stats.items()}

    got = fit_probability_threshold(samples(on_gpu), 8.0)
    want = fit_probability_threshold(samples(on_cpu), 8.0)
    assert got["tau"] == want["tau"] and got["threshold_code"] == want["threshold_code"]
    assert math.isclose(got["squared_error"], want["squared_error"], rel_tol=1e-3)


@pytest.mark.parametrize("rotation", ["none", "hadamard"])
def test_runtime_measures_the_key_mean(rotation):
    """begin -> per-layer, per-step accumulation -> finish: the sidecar value is the FP64 mean
    rounded once to BF16, the active shift the same mean in the write path's basis."""
    pytest.importorskip("vllm")
    from nvfp4_vllm.runtime import LayerRuntime, sylvester_hadamard

    layers, heads = 2, 2
    runtime = LayerRuntime(num_layers=layers, num_slots=4, num_heads=8, num_kv_heads=heads, head_dim=128,
                           device="cuda", query_terms=2, rotation=rotation)
    with pytest.raises(ValueError):
        runtime.finish_key_shift_measurement()
    runtime.begin_key_shift_measurement()
    gen = torch.Generator().manual_seed(5)
    seen = [[], []]
    for tokens in (700, 33, 1):
        for layer in range(layers):
            key = (torch.randn(tokens + 5, heads * 128, generator=gen) + 0.25 * layer).to(torch.bfloat16).cuda()
            runtime.measure_keys(layer, key, tokens)  # rows past `tokens` are padding
            seen[layer].append(key[:tokens].view(tokens, heads, 128))
    assert runtime.key_shift_tokens == 734
    measured = runtime.finish_key_shift_measurement()
    mean = torch.stack([torch.cat(rows).double().mean(dim=0) for rows in seen])
    assert torch.equal(measured, mean.to(torch.bfloat16))
    if rotation == "none":
        assert torch.equal(runtime.active_key_shift, measured)
    else:
        rotated = (mean @ sylvester_hadamard(128, "cuda").T).float()
        assert torch.allclose(runtime.active_key_shift, rotated, rtol=0, atol=1e-6)
        assert runtime.active_key_shift.dtype is torch.float32
    assert runtime.key_shift_sum is None and runtime.key_shift_enabled
    runtime.measure_keys(0, key, 1)  # a no-op once the measurement is over


def test_probability_calibration_collector_end_to_end():
    """The collector's hook on a stand-in attention layer: BF16 Q/K of one unchunked prefill in,
    per-position per-code error sums out, and a threshold fitted from them. The scores go through
    the CUDA statistic; the oracle gives the same fit."""
    pytest.importorskip("vllm")
    import types

    from nvfp4_vllm.probability_calibration import ProbabilityCalibration, fit_probability_threshold

    tokens, heads, kv_heads, dim = 640, 8, 2, 128
    gen = torch.Generator(device="cuda").manual_seed(21)
    query = (2.5 * torch.randn(tokens + 7, heads * dim, generator=gen, device="cuda")).to(torch.bfloat16)
    key = (2.5 * torch.randn(tokens + 7, kv_heads * dim, generator=gen, device="cuda")).to(torch.bfloat16)
    module = types.SimpleNamespace(num_heads=heads, num_kv_heads=kv_heads, head_size=dim)
    collector = ProbabilityCalibration(tokens, 8.0, samples=3)
    collector.expected_layers = 1
    collector.observe(module, (query, key), {})
    with pytest.raises(RuntimeError):
        collector.observe(module, (query, key), {})  # one prefill per layer
    samples = collector.finish()
    assert [s["position"] for s in samples] == collector.positions == [128, 383, 639]
    for sample in samples:
        groups = heads * (sample["position"] // 128) * 128 // 16
        assert sum(bucket["groups"] for bucket in sample["codes"].values()) == groups
    report = fit_probability_threshold([samples], 8.0)

    # the same samples from the CPU oracle
    q = query[:tokens].float().cpu().reshape(tokens, kv_heads, heads // kv_heads, dim)
    k = key[:tokens].float().cpu().reshape(tokens, kv_heads, dim)
    want = []
    for position in collector.positions:
        scores = torch.einsum("hrd,thd->hrt", q[position], k[:position + 1]).reshape(heads, position + 1)
        stats = calibration_oracle.probability_scale_statistics(scores, fp4_tokens=(position // 128) * 128, head_dim=dim,
                                                                probability_multiplier=8.0)
        want.append({"position": position, "codes": {
            code: {"groups": b["groups"], "error_sum": {"6": b["error_sum"][0], "2": b["error_sum"][3]}}
            for code, b in stats.items()}})
    expected = fit_probability_threshold([want], 8.0)
    assert report["tau"] == expected["tau"] and report["groups"] == expected["groups"]
    assert math.isclose(report["squared_error"], expected["squared_error"], rel_tol=1e-3)
    with pytest.raises(ValueError):
        ProbabilityCalibration(tokens, 8.0, samples=3).observe(module, (query[:100], key[:100]), {})
