"""CPU restatement of the calibration statistic of OpenBitSys/BitDecoding-FP4.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``; no product code may import this module.
Pinned to the reference by ``tests/golden/calibration_vectors.json``, which
``tests/golden/make_calibration_golden.py`` produced by running the reference's own
``online_probability_scale_statistics`` (src/nvfp4_decode_kernel/reference.py:758-871) on seeded
scores in this container.
"""

from __future__ import annotations

import torch

from . import nvfp4_oracle as base

DIVISORS = (6.0, 4.0, 3.0, 2.0)  # tie-break order of the reference's "e2m1_max_grid" rungs


def probability_scale_statistics(scores: torch.Tensor, *, fp4_tokens: int, head_dim: int, sink_tokens: int = 16,
                                 probability_multiplier: float = 1.0) -> dict:
    """Per-E4M3-code error statistics of the FP4 probability operand for one query position.

    ``scores`` is FP32 ``[heads, tokens]`` (unscaled QK). The FP4 prefix is walked page by page,
    newest first, as decode does: a page's probabilities are formed against the maximum over that
    page, every newer page and the tokens past the prefix; the first ``sink_tokens`` positions of
    page 0 are masked. Each 16-token group, times ``probability_multiplier``, is priced under the
    scale divisors 6, 4, 3, 2 (scale = max/divisor, stored as E4M3; codes from the unrounded scale)
    and the squared errors are summed per E4M3 code of the group maximum
    (src/nvfp4_decode_kernel/reference.py:787-846).
    Returns ``{code: {"groups", "winner_counts": [4], "error_sum": [4], "oracle_error_sum"}}``.
    """
    heads, tokens = scores.shape
    page = base.PAGE
    scaled = scores.float() * float(head_dim ** -0.5)
    pages = scaled[:, :fp4_tokens].reshape(heads, -1, page).clone()
    if sink_tokens:
        pages[:, 0, :sink_tokens] = -torch.inf
    running = torch.full((heads,), -torch.inf)
    if fp4_tokens < tokens:
        running = scaled[:, fp4_tokens:].amax(dim=-1)
    held = torch.empty(heads, pages.shape[1])
    for index in range(pages.shape[1] - 1, -1, -1):  # newest page first
        running = torch.maximum(running, pages[:, index].amax(dim=-1))
        held[:, index] = running
    held = torch.where(torch.isfinite(held), held, torch.zeros_like(held))
    probability = torch.exp(pages - held[..., None])
    probability = torch.where(torch.isfinite(pages), probability, torch.zeros_like(probability))
    groups = (probability * probability_multiplier).reshape(-1, 16)
    maximum = groups.amax(dim=-1, keepdim=True)
    code = base.e4m3_bytes(maximum.squeeze(-1)).long()
    errors = []
    for divisor in DIVISORS:
        raw = maximum * float(1.0 / divisor)
        stored = base.e4m3_round(raw)
        magnitude = base.e2m1_decode(base.e2m1_codes(groups / raw.clamp_min(1.0e-30)))
        errors.append((magnitude * stored - groups).square().sum(dim=-1))
    error = torch.stack(errors, dim=-1)
    winner = error.argmin(dim=-1)
    best = error.gather(-1, winner[:, None]).squeeze(-1)
    out = {}
    for value in torch.unique(code).tolist():
        pick = code == value
        out[int(value)] = {
            "groups": int(pick.sum()),
            "winner_counts": [int((winner[pick] == d).sum()) for d in range(len(DIVISORS))],
            "error_sum": [float(error[pick, d].double().sum()) for d in range(len(DIVISORS))],
            "oracle_error_sum": float(best[pick].double().sum()),
        }
    return out
