"""The calibration statistic of src/nvfp4_decode_kernel/reference.py that callers outside the
package use (``online_probability_scale_statistics``, :758-871 of OpenBitSys/BitDecoding-FP4),
computed on the GPU by ``bdfp4_probability_statistics``.

Only that function lives here. The reference module's CPU model of the quantizer and of
attention is what this repository's test oracle restates; the product has no CPU path.
"""

from __future__ import annotations

import math

import torch

import bdfp4

PAGE_SIZE = 128
DIVISORS = (6, 4, 3, 2)  # the "e2m1_max_grid" rungs, in tie-break order


def online_probability_scale_statistics(scores: torch.Tensor, *, fp4_tokens: int, head_dim: int,
                                        sink_tokens: int = 16, page_size: int = PAGE_SIZE,
                                        probability_multiplier: float = 1.0) -> dict:
    """Exact probability-scale errors of one query position, aggregated by the E4M3 code of each
    16-value group's maximum.

    ``scores`` is a CUDA ``[heads, tokens]`` tensor of unscaled Q.K products (converted to FP32).
    The FP4 prefix ``scores[:, :fp4_tokens]`` is walked newest page first, as decode walks it, so
    a page's probabilities are taken against the maximum the online softmax holds when it gets
    there; the first ``sink_tokens`` positions of page 0 are masked. Returns the reference's
    dictionary: totals plus ``by_amax_e4m3_code`` with, per code, ``groups``, ``winner_counts``,
    ``error_sum`` (keys "6", "4", "3", "2") and ``oracle_error_sum``."""
    if scores.ndim != 2:
        raise ValueError("scores must have shape [heads, tokens]")
    if not scores.is_cuda:
        raise RuntimeError("online_probability_scale_statistics runs on the GPU; pass CUDA scores")
    if page_size != PAGE_SIZE:
        raise NotImplementedError("only 128-token pages are built")
    heads, tokens = scores.shape
    if fp4_tokens <= 0 or fp4_tokens > tokens or fp4_tokens % page_size:
        raise ValueError("fp4_tokens must be positive, page aligned, and in range")
    if not 0 <= sink_tokens <= fp4_tokens:
        raise ValueError("sink tokens must lie inside the FP4 prefix")
    if not math.isfinite(probability_multiplier) or not 0 < probability_multiplier <= 448:
        raise ValueError("probability_multiplier must be finite and between 0 and 448")
    device = scores.device
    scores = scores.float().contiguous()
    pages = fp4_tokens // page_size
    page_max = torch.empty(heads * (pages + 1), dtype=torch.float32, device=device)
    counts = torch.zeros(256, dtype=torch.int64, device=device)
    winners = torch.zeros(256, len(DIVISORS), dtype=torch.int64, device=device)
    errors = torch.zeros(256, len(DIVISORS), dtype=torch.float64, device=device)
    oracle = torch.zeros(256, dtype=torch.float64, device=device)
    bdfp4.probability_statistics(
        scores, fp4_tokens=fp4_tokens, softmax_scale=float(head_dim ** -0.5), sink_tokens=min(sink_tokens, page_size),
        multiplier=float(probability_multiplier), page_max_scratch=page_max, group_counts=counts,
        winner_counts=winners, error_sums=errors, oracle_sums=oracle, stream=bdfp4.current_stream(device))
    counts, winners, errors, oracle = counts.tolist(), winners.tolist(), errors.tolist(), oracle.tolist()
    by_code = {
        str(code): {
            "groups": counts[code],
            "winner_counts": {str(d): winners[code][i] for i, d in enumerate(DIVISORS)},
            "error_sum": {str(d): errors[code][i] for i, d in enumerate(DIVISORS)},
            "oracle_error_sum": oracle[code],
        }
        for code in range(256) if counts[code]
    }
    return {
        "group_count": sum(counts),
        "divisors": list(DIVISORS),
        "winner_counts": {str(d): sum(row[i] for row in winners) for i, d in enumerate(DIVISORS)},
        "error_sum": {str(d): math.fsum(row[i] for row in errors) for i, d in enumerate(DIVISORS)},
        "oracle_error_sum": math.fsum(oracle),
        "by_amax_e4m3_code": by_code,
    }
