"""Calibration of tau, the threshold of the probability operand's two-scale rule.

During decode a group of sixteen probabilities is stored with scale ``max/2`` when its maximum is at
most tau and with ``max/6`` otherwise. Which maxima are better served by ``max/2`` is an empirical
question about a model's attention, so tau is fitted: while one long prefill runs, a few query
positions are taken, every attention layer's BF16 scores at those positions are priced group by group
under both scales on the GPU (``bdfp4_probability_statistics``), and the squared errors are summed per
E4M3 code of the group maximum. Since the rule is a cut on that code, the fit is a one-dimensional
search over cuts; leaving one query position out at a time says how stable the cut is.

The public names, the shape of a sample and every key of the report are those of
src/nvfp4_vllm/probability_calibration.py of OpenBitSys/BitDecoding-FP4, so the two are
interchangeable for callers; ``tests/test_calibration_golden.py`` holds this fit to that module's
outputs value for value.
"""

from __future__ import annotations

import math
import struct
from dataclasses import dataclass, field

CODES = 126          # E4M3 codes a group maximum can take here: 0 .. 125
HALF, SIXTH = "2", "6"  # the two divisors, as the statistics name them


def threshold_for_code(code: int) -> float:
    """tau such that ``x <= tau`` (FP32) holds exactly for the values that round to an E4M3 code of at
    most ``code``. Rounding is to nearest with ties to the even code, so the boundary is the midpoint
    to the next code, owned by whichever of the two codes is even: under an odd ``code`` the midpoint
    belongs to its neighbour and tau is the FP32 number just below it. ``-1`` switches ``max/2`` off."""
    if code == -1:
        return 0.0
    if not 0 <= code < CODES:
        raise ValueError("threshold code must be in [-1, 125]")

    def value(c: int) -> float:  # bias 7, three mantissa bits, subnormals under 2^-6
        exponent, mantissa = divmod(c, 8)
        return math.ldexp(mantissa, -9) if exponent == 0 else math.ldexp(8 + mantissa, exponent - 10)

    midpoint = (value(code) + value(code + 1)) / 2
    if code % 2 == 0:
        return midpoint
    (bits,) = struct.unpack("<I", struct.pack("<f", midpoint))
    return struct.unpack("<f", struct.pack("<I", bits - 1))[0]


@dataclass
class _Tally:
    """Group counts and summed squared errors under each scale, one slot per E4M3 code."""

    groups: list = field(default_factory=lambda: [0] * CODES)
    error: dict = field(default_factory=lambda: {HALF: [0.0] * CODES, SIXTH: [0.0] * CODES})
    seen: set = field(default_factory=set)

    def add(self, sample: dict) -> None:
        for code, bucket in sample["codes"].items():
            code = int(code)
            sums = bucket["error_sum"]
            ok = 0 <= code < CODES and bucket["groups"] >= 1 and all(
                math.isfinite(sums[d]) and sums[d] >= 0 for d in (HALF, SIXTH))
            if not ok:
                raise ValueError("invalid probability calibration statistics")
            self.seen.add(code)
            self.groups[code] += bucket["groups"]
            for d in (HALF, SIXTH):
                self.error[d][code] += sums[d]

    def without(self, other: "_Tally") -> "_Tally":
        rest = _Tally(seen=set(self.seen))
        rest.groups = [a - b for a, b in zip(self.groups, other.groups)]
        for d in (HALF, SIXTH):
            rest.error[d] = [a - b for a, b in zip(self.error[d], other.error[d])]
        return rest

    def cost(self, cut: int) -> float:
        """Summed error when codes up to ``cut`` take max/2 and the others max/6."""
        return math.fsum(self.error[HALF][:cut + 1] + self.error[SIXTH][cut + 1:])

    def best_cut(self) -> int:
        """The lowest cut with the least cost; -1 (max/6 everywhere) wins ties with everything."""
        cuts = range(-1, max(self.seen) + 1)
        costs = [self.cost(cut) for cut in cuts]
        return cuts[costs.index(min(costs))]


def fit_probability_threshold(worker_samples: list[list[dict]], multiplier: float) -> dict:
    """The report of a calibration run: tau over all samples and, for every query position, the tau
    fitted without it together with the error that tau leaves on it.

    ``worker_samples[w]`` are worker ``w``'s samples ``{"position", "codes": {code: {"groups",
    "error_sum": {"2", "6"}}}}`` (tensor-parallel workers see different heads of the same positions).
    Errors are measured on ``multiplier x probability`` and reported divided by ``multiplier**2``."""
    if not (math.isfinite(multiplier) and multiplier > 0):
        raise ValueError("probability multiplier must be positive and finite")
    overall, per_position = _Tally(), {}
    for sample in (s for worker in worker_samples for s in worker):
        per_position.setdefault(sample["position"], _Tally()).add(sample)
        overall.add(sample)
    if len(per_position) < 2:
        raise ValueError("tau calibration needs at least two query positions")
    if any(not tally.seen for tally in per_position.values()):
        raise ValueError("invalid probability calibration statistics")
    unit = multiplier ** 2
    cut = overall.best_cut()
    folds = []
    for position in sorted(per_position):
        held = per_position[position]
        trained = overall.without(held).best_cut()
        folds.append({"position": position, "tau": threshold_for_code(trained),
                      "squared_error": held.cost(trained) / unit})
    return {
        "tau": threshold_for_code(cut),
        "c": multiplier,
        "rule": "max(p) <= tau / c",
        "threshold_code": cut,
        "samples": len(per_position),
        "groups": sum(overall.groups),
        "squared_error": overall.cost(cut) / unit,
        "amax6_squared_error": overall.cost(-1) / unit,
        "validation": "leave_one_query_position_out",
        "folds": folds,
        "source": "BF16 Q/K, reverse-page online softmax, 16-value probability groups",
    }


class ProbabilityCalibration:
    """Collects the per-code error sums of one unchunked prefill.

    ``samples`` query positions are spaced evenly from 128 to the last token. :meth:`install` hooks
    every attention layer of a model; each layer's forward then calls :meth:`observe` once with its
    Q and K, and :meth:`finish` hands back one sample per position once every layer has reported.
    Only the sums are kept, never scores."""

    def __init__(self, tokens: int, multiplier: float, samples: int = 8):
        if tokens < 256 or not 2 <= samples <= tokens - 128:
            raise ValueError("tau calibration needs at least 256 tokens and 2..tokens-128 samples")
        if not (math.isfinite(multiplier) and 0 < multiplier <= 448):
            raise ValueError("probability multiplier must be finite and between 0 and 448")
        self.tokens, self.multiplier = tokens, multiplier
        span = tokens - 129
        self.positions = [128 + (index * span) // (samples - 1) for index in range(samples)]
        self.samples = {position: {"position": position, "codes": {}} for position in self.positions}
        self.handles: list = []
        self.seen: set = set()
        self.expected_layers = 0

    def install(self, model) -> None:
        """Hook every attention layer of ``model``; the engine must run eagerly for hooks to fire."""
        from vllm.model_executor.layers.attention.attention import Attention

        layers = [module for module in model.modules() if isinstance(module, Attention)]
        if not layers:
            raise ValueError("no attention layers found for probability calibration")
        try:
            for layer in layers:
                self.handles.append(layer.register_forward_pre_hook(self.observe, with_kwargs=True))
        except BaseException:
            self.close()
            raise
        self.expected_layers = len(layers)

    def _scores(self, query, key, position: int, heads: int, kv_heads: int, dim: int):
        """FP32 scores ``[heads, position + 1]`` of the query at ``position`` against every key so far."""
        import torch

        group = heads // kv_heads
        q = query[position].float().view(kv_heads, group, dim)
        k = key[:position + 1].view(position + 1, kv_heads, dim)
        return torch.einsum("hrd,thd->hrt", q, k).reshape(heads, position + 1)

    def observe(self, module, args, kwargs) -> None:
        import torch

        from nvfp4_decode_kernel.reference import online_probability_scale_statistics

        if id(module) in self.seen:
            raise RuntimeError("tau calibration requires one complete prefill per attention layer")
        query = args[0] if len(args) > 0 else kwargs["query"]
        key = args[1] if len(args) > 1 else kwargs["key"]
        if min(query.shape[0], key.shape[0]) < self.tokens:
            raise ValueError("tau calibration requires an unchunked prefill")
        heads, kv_heads, dim = module.num_heads, module.num_kv_heads, module.head_size
        if query.dtype is not torch.bfloat16 or key.dtype is not torch.bfloat16 or heads % kv_heads:
            raise ValueError("tau calibration requires BF16 Q/K and grouped-query attention")
        query = query[:self.tokens].reshape(self.tokens, heads, dim)
        key = key[:self.tokens].reshape(self.tokens, kv_heads, dim).float()
        matmul = torch.backends.cuda.matmul
        tf32, matmul.allow_tf32 = matmul.allow_tf32, False  # these scores are the FP32 reference
        try:
            for position in self.positions:
                stats = online_probability_scale_statistics(
                    self._scores(query, key, position, heads, kv_heads, dim), fp4_tokens=position // 128 * 128,
                    head_dim=dim, probability_multiplier=self.multiplier)
                codes = self.samples[position]["codes"]
                for code, bucket in stats["by_amax_e4m3_code"].items():
                    entry = codes.setdefault(code, {"groups": 0, "error_sum": {HALF: 0.0, SIXTH: 0.0}})
                    entry["groups"] += bucket["groups"]
                    for d in (HALF, SIXTH):
                        entry["error_sum"][d] += bucket["error_sum"][d]
        finally:
            matmul.allow_tf32 = tf32
        self.seen.add(id(module))

    def finish(self) -> list[dict]:
        if len(self.seen) != self.expected_layers:
            raise RuntimeError("not every attention layer supplied probability calibration samples")
        return list(self.samples.values())

    def close(self) -> None:
        while self.handles:
            self.handles.pop().remove()
