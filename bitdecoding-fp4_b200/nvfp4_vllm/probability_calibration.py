"""Fit the probability-scale threshold tau from a bounded sample of one long prefill
(src/nvfp4_vllm/probability_calibration.py of OpenBitSys/BitDecoding-FP4).

The decode kernel scales a group of sixteen probabilities by ``max/2`` when the group's maximum is
at most tau and by ``max/6`` otherwise. For a few query positions of an unchunked prefill the
collector forms the BF16 Q.K scores of every attention layer, and a CUDA kernel
(``bdfp4_probability_statistics``) prices every FP4-prefix group under both divisors, bucketed by
the E4M3 code of the group's maximum. Tau is then the code boundary that minimises the summed
error, validated by leaving one query position out at a time.
"""

from __future__ import annotations

import math
import struct


def _e4m3_value(code: int) -> float:
    """Value of a non-negative E4M3 code (bias 7, three mantissa bits, subnormals below 2^-6)."""
    exponent, mantissa = code >> 3, code & 7
    if exponent == 0:
        return mantissa * 2.0 ** -9
    return (8 + mantissa) * 2.0 ** (exponent - 10)


def _float32_below(value: float) -> float:
    bits = struct.unpack("<I", struct.pack("<f", value))[0]
    return struct.unpack("<f", struct.pack("<I", bits - 1))[0]


def threshold_for_code(code: int) -> float:
    """The largest FP32 ``tau`` such that ``x <= tau`` holds exactly for the values whose E4M3
    round-to-nearest-even code is at most ``code``. The cut is the midpoint to the next code; a
    tie at the midpoint rounds to the even code, so below an odd ``code`` the midpoint itself
    belongs to the next code and the cut is the FP32 value just under it
    (src/nvfp4_vllm/probability_calibration.py:14-25). ``-1`` means no group takes ``max/2``."""
    if code == -1:
        return 0.0
    if not 0 <= code < 126:
        raise ValueError("threshold code must be in [-1, 125]")
    midpoint = 0.5 * (_e4m3_value(code) + _e4m3_value(code + 1))
    return _float32_below(midpoint) if code & 1 else midpoint


def _merged(samples) -> dict[int, dict[str, float]]:
    """Per-code totals of several samples: group count and the error sums under /2 and /6."""
    totals: dict[int, dict[str, float]] = {}
    for sample in samples:
        for code, bucket in sample["codes"].items():
            entry = totals.setdefault(int(code), {"groups": 0, "2": 0.0, "6": 0.0})
            entry["groups"] += bucket["groups"]
            entry["2"] += bucket["error_sum"]["2"]
            entry["6"] += bucket["error_sum"]["6"]
    return totals


def _cost(buckets: dict, cut: int) -> float:
    """Summed squared error when codes up to ``cut`` use max/2 and the rest max/6."""
    return math.fsum(bucket["2"] if code <= cut else bucket["6"] for code, bucket in buckets.items())


def _argmin_cut(buckets: dict) -> int:
    best, best_cost = -1, _cost(buckets, -1)
    for cut in range(0, max(buckets) + 1):
        cost = _cost(buckets, cut)
        if cost < best_cost:
            best, best_cost = cut, cost
    return best


def fit_probability_threshold(worker_samples: list[list[dict]], multiplier: float) -> dict:
    """Tau from every worker's samples, plus a leave-one-query-position-out check.

    ``worker_samples[w]`` is worker ``w``'s list of ``{"position", "codes": {code: {"groups",
    "error_sum": {"2", "6"}}}}``; errors are in units of (multiplier x probability)^2 and reported
    divided by ``multiplier**2`` (src/nvfp4_vllm/probability_calibration.py:46-87)."""
    if not math.isfinite(multiplier) or multiplier <= 0:
        raise ValueError("probability multiplier must be positive and finite")
    by_position: dict[int, list[dict]] = {}
    for worker in worker_samples:
        for sample in worker:
            by_position.setdefault(sample["position"], []).append(sample)
    if len(by_position) < 2:
        raise ValueError("tau calibration needs at least two query positions")
    held_out = {position: _merged(samples) for position, samples in by_position.items()}
    for buckets in held_out.values():
        bad = not buckets
        for code, bucket in buckets.items():
            bad = bad or not 0 <= code < 126 or bucket["groups"] < 1
            bad = bad or any(not math.isfinite(bucket[d]) or bucket[d] < 0 for d in ("2", "6"))
        if bad:
            raise ValueError("invalid probability calibration statistics")
    total = _merged(sample for worker in worker_samples for sample in worker)
    cut = _argmin_cut(total)
    folds = []
    for position in sorted(held_out):
        held = held_out[position]
        training = {code: {name: value - held.get(code, {}).get(name, 0) for name, value in bucket.items()}
                    for code, bucket in total.items()}
        training_cut = _argmin_cut(training)
        folds.append({"position": position, "tau": threshold_for_code(training_cut),
                      "squared_error": _cost(held, training_cut) / multiplier ** 2})
    return {
        "tau": threshold_for_code(cut), "c": multiplier, "rule": "max(p) <= tau / c", "threshold_code": cut,
        "samples": len(by_position), "groups": sum(bucket["groups"] for bucket in total.values()),
        "squared_error": _cost(total, cut) / multiplier ** 2,
        "amax6_squared_error": math.fsum(bucket["6"] for bucket in total.values()) / multiplier ** 2,
        "validation": "leave_one_query_position_out", "folds": folds,
        "source": "BF16 Q/K, reverse-page online softmax, 16-value probability groups",
    }


class ProbabilityCalibration:
    """Watches one unchunked prefill and keeps only per-code error sums.

    ``samples`` query positions are spread evenly over ``[128, tokens)``; for each, every attention
    layer contributes the statistics of its heads' score rows against all earlier keys."""

    def __init__(self, tokens: int, multiplier: float, samples: int = 8):
        if tokens < 256 or not 2 <= samples <= tokens - 128:
            raise ValueError("tau calibration needs at least 256 tokens and 2..tokens-128 samples")
        if not math.isfinite(multiplier) or not 0 < multiplier <= 448:
            raise ValueError("probability multiplier must be finite and between 0 and 448")
        self.tokens = tokens
        self.multiplier = multiplier
        self.positions = [128 + index * (tokens - 129) // (samples - 1) for index in range(samples)]
        self.samples = {position: {"position": position, "codes": {}} for position in self.positions}
        self.handles = []
        self.seen = set()
        self.expected_layers = 0

    def install(self, model) -> None:
        """Hook every attention layer of ``model`` (needs an eager engine, so that hooks run)."""
        from vllm.model_executor.layers.attention.attention import Attention

        try:
            for module in model.modules():
                if isinstance(module, Attention):
                    self.handles.append(module.register_forward_pre_hook(self.observe, with_kwargs=True))
            self.expected_layers = len(self.handles)
            if not self.expected_layers:
                raise ValueError("no attention layers found for probability calibration")
        except BaseException:
            self.close()
            raise

    def observe(self, module, args, kwargs) -> None:
        import torch

        from nvfp4_decode_kernel.reference import online_probability_scale_statistics

        if id(module) in self.seen:
            raise RuntimeError("tau calibration requires one complete prefill per attention layer")
        query = args[0] if args else kwargs["query"]
        key = args[1] if len(args) > 1 else kwargs["key"]
        if query.shape[0] < self.tokens or key.shape[0] < self.tokens:
            raise ValueError("tau calibration requires an unchunked prefill")
        heads, kv_heads, dim = module.num_heads, module.num_kv_heads, module.head_size
        if query.dtype != torch.bfloat16 or key.dtype != torch.bfloat16 or heads % kv_heads:
            raise ValueError("tau calibration requires BF16 Q/K and grouped-query attention")
        query = query[:self.tokens].reshape(self.tokens, heads, dim)
        key = key[:self.tokens].reshape(self.tokens, kv_heads, dim).float()
        tf32 = torch.backends.cuda.matmul.allow_tf32
        try:
            torch.backends.cuda.matmul.allow_tf32 = False  # the scores are an FP32 reference
            for position in self.positions:
                rows = query[position].float().reshape(kv_heads, heads // kv_heads, dim)
                scores = torch.einsum("hrd,thd->hrt", rows, key[:position + 1]).reshape(heads, position + 1)
                stats = online_probability_scale_statistics(
                    scores, fp4_tokens=(position // 128) * 128, head_dim=dim,
                    probability_multiplier=self.multiplier)
                into = self.samples[position]["codes"]
                for code, bucket in stats["by_amax_e4m3_code"].items():
                    entry = into.setdefault(code, {"groups": 0, "error_sum": {"2": 0.0, "6": 0.0}})
                    entry["groups"] += bucket["groups"]
                    entry["error_sum"]["2"] += bucket["error_sum"]["2"]
                    entry["error_sum"]["6"] += bucket["error_sum"]["6"]
        finally:
            torch.backends.cuda.matmul.allow_tf32 = tf32
        self.seen.add(id(module))

    def finish(self) -> list[dict]:
        if len(self.seen) != self.expected_layers:
            raise RuntimeError("not every attention layer supplied probability calibration samples")
        return list(self.samples.values())

    def close(self) -> None:
        for handle in self.handles:
            handle.remove()
        self.handles.clear()
