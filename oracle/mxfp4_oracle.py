"""CPU oracle of the MXFP4 format (E2M1 codes, one E8M0 power-of-two scale per 32 values).
TEST INFRASTRUCTURE: only tests may import it; the product never does, and has no MXFP4 kernel yet.

Restates mxfp4_quantize and mxfp4_probability_quantize of OpenBitSys/BitDecoding-FP4
(src/nvfp4_decode_kernel/reference.py:262-358) and is pinned bit-exactly against outputs of those
functions in tests/golden/mxfp4_vectors.npz (made by tests/golden/make_mxfp4_golden.py).

    ocp       exponent = floor(log2(amax)) - 2, clamped to the E8M0 range [-127, 127]
    round_up  ocp + 1 when amax > 6 * 2^ocp (the smallest exponent keeping amax within E2M1's 6)
    search    ocp + 1 when it reconstructs the group with strictly less squared error
    an all-zero group takes exponent -127 (E8M0 has no zero); the stored byte is exponent + 127
"""

from __future__ import annotations

import torch

from . import nvfp4_oracle as base

GROUP = 32
RULES = ("ocp", "round_up", "search")
EXPONENT_MIN, EXPONENT_MAX = -127, 127


def _power_of_two(exponent: torch.Tensor) -> torch.Tensor:
    return torch.ldexp(torch.ones(exponent.shape, dtype=torch.float32), exponent)


def _on_scale(groups: torch.Tensor, exponent: torch.Tensor):
    """Codes of ``groups`` on the scale ``2**exponent`` and the values they read back as."""
    scale = _power_of_two(exponent)
    codes = base.e2m1_codes(groups / scale)
    return codes, base.e2m1_decode(codes) * scale


def ocp_exponent(amax: torch.Tensor) -> torch.Tensor:
    """floor(log2(amax)) - 2 without a logarithm: amax = m * 2^k with m in [0.5, 1) gives
    floor(log2(amax)) = k - 1 (reference.py:299-306)."""
    _, k = torch.frexp(amax.float())
    exponent = (k.to(torch.int32) - 3).clamp(EXPONENT_MIN, EXPONENT_MAX)
    return torch.where(amax > 0, exponent, torch.full_like(exponent, EXPONENT_MIN))


def quantize_last_axis(x: torch.Tensor, rule: str = "ocp"):
    """``[..., n]`` (n % 32 == 0) -> (codes u8 ``[..., n]``, E8M0 bytes ``[..., n/32]``, winner
    int64 ``[..., n/32]``: 0 for the OCP exponent, 1 for the one above it)."""
    if rule not in RULES:
        raise ValueError(f"rule must be one of {RULES}, got {rule!r}")
    groups = x.float().reshape(*x.shape[:-1], x.shape[-1] // GROUP, GROUP)
    amax = groups.abs().amax(dim=-1, keepdim=True)
    exponent = ocp_exponent(amax)
    codes, values = _on_scale(groups, exponent)
    winner = torch.zeros_like(exponent, dtype=torch.int64)
    if rule != "ocp":
        above = (exponent + 1).clamp(max=EXPONENT_MAX)
        above_codes, above_values = _on_scale(groups, above)
        if rule == "round_up":
            choose = amax > 6.0 * _power_of_two(exponent)
        else:
            choose = (base._fma_squares(above_values - groups) < base._fma_squares(values - groups))[..., None]
        winner = choose.to(torch.int64)
        exponent = torch.where(choose, above, exponent)
        codes = torch.where(choose, above_codes, codes)
    return codes.reshape(x.shape), (exponent + 127).to(torch.uint8).squeeze(-1), winner.squeeze(-1)


def dequantize_last_axis(codes: torch.Tensor, scale_bytes: torch.Tensor) -> torch.Tensor:
    groups = base.e2m1_decode(codes).reshape(*codes.shape[:-1], codes.shape[-1] // GROUP, GROUP)
    scale = _power_of_two(scale_bytes.to(torch.int32) - 127)
    return (groups * scale[..., None]).reshape(codes.shape)


def probability_quantize(p: torch.Tensor):
    """The probability operand in MXFP4 (reference.py:331-358): start from ``round_up`` and take the
    exponent below it when that lowers ``mass^2 / 32 + sum of squared errors``, the error sums formed
    by a five-step pairwise (butterfly) reduction and the final combination in FP64 rounded to FP32.
    Returns (values the PV product sees, E8M0 bytes)."""
    codes, scale_bytes, _ = quantize_last_axis(p, "round_up")
    groups = p.float().reshape(*p.shape[:-1], p.shape[-1] // GROUP, GROUP)
    baseline = dequantize_last_axis(codes, scale_bytes).reshape(groups.shape)
    exponent = scale_bytes.to(torch.int32)[..., None] - 127
    below = (exponent - 1).clamp(min=EXPONENT_MIN)
    _, rival = _on_scale(groups, below)

    def cost(values):
        difference = values - groups
        squares, mass = difference.square(), difference
        for _ in range(5):
            squares = squares[..., 0::2] + squares[..., 1::2]
            mass = mass[..., 0::2] + mass[..., 1::2]
        return ((mass / 32).double() * mass.double() + squares.double()).float()

    choose = cost(rival) < cost(baseline)
    values = torch.where(choose, rival, baseline).reshape(p.shape)
    chosen = torch.where(choose, below, exponent).squeeze(-1)
    return values, (chosen + 127).to(torch.uint8)
