"""Configuration of the FP4 softmax-probability operand.

The decode kernel quantizes each group of sixteen probabilities with scale ``amax/2`` when the
group's maximum is at most a threshold tau and ``amax/6`` otherwise, optionally on
probabilities pre-multiplied by 8 (``_c8``; the LSE is corrected for it). Environment variables
and defaults mirror src/nvfp4_decode_kernel/p_scale.py of OpenBitSys/BitDecoding-FP4; unlike
there, the mode and tau are arguments of the kernel launch rather than constants baked in at
import, so the values read here are only the defaults.
"""

from __future__ import annotations

import math
import os
from collections.abc import Mapping

DEFAULT_P_SCALE_TAU = 21.0 / 1024.0  # halfway between the E4M3 neighbours 20/1024 and 22/1024
DEFAULT_P_SCALE_MODE = "amax2_or_amax6_c8"
P_SCALE_MODES: dict[str, tuple[float, ...]] = {
    "amax6": (6.0,),
    "two_level": (6.0,),
    "amax4": (4.0,),
    "amax3": (3.0,),
    "amax2": (2.0,),
    "e2m1_max_grid": (6.0, 4.0, 3.0, 2.0),
    "amax2_or_amax6": (2.0, 6.0),
    "amax2_or_amax6_c8": (2.0, 6.0),
}
# modes this build has kernels for
BUILT_P_SCALE_MODES = ("amax6", "amax2_or_amax6", "amax2_or_amax6_c8")
_LEGACY = {"e4m3_amax_code10_threshold": "amax2_or_amax6"}


def resolve_p_scale_tau(environment: Mapping[str, str] | None = None) -> float:
    """tau from ``NVFP4_P_SCALE_TAU`` (scaled-probability units), default 21/1024."""
    env = os.environ if environment is None else environment
    tau = float(env.get("NVFP4_P_SCALE_TAU", DEFAULT_P_SCALE_TAU))
    if not (math.isfinite(tau) and 0 <= tau <= 448):
        raise ValueError("NVFP4_P_SCALE_TAU must be finite and between 0 and 448")
    return tau


P_SMALL_GROUP_AMAX = resolve_p_scale_tau()


def p_scale_is_amax2_or_amax6(mode: str) -> bool:
    return _LEGACY.get(mode, mode) in ("amax2_or_amax6", "amax2_or_amax6_c8")


def resolve_p_scale_environment(environment: Mapping[str, str] | None = None) -> tuple[str, float, bool]:
    """``(mode, fixed_divisor, searches_grid)`` from ``NVFP4_P_SCALE_MODE`` / ``NVFP4_P_SCALE_DIVISOR``.

    With neither set the mode is the default. A divisor alone selects ``amax<d>``; a mode and a
    divisor that disagree raise. Adaptive modes report 6 as a placeholder divisor.
    """
    env = os.environ if environment is None else environment
    mode = env.get("NVFP4_P_SCALE_MODE")
    divisor_text = env.get("NVFP4_P_SCALE_DIVISOR")
    if mode is None and divisor_text is None:
        mode = DEFAULT_P_SCALE_MODE
    if mode is None:
        try:
            divisor = float(divisor_text)
        except ValueError:
            divisor = math.nan
        if divisor not in (2.0, 3.0, 4.0, 6.0):
            raise ValueError(f"NVFP4_P_SCALE_DIVISOR must be 2, 3, 4, or 6, got {divisor_text!r}")
        return f"amax{int(divisor)}", divisor, False
    mode = _LEGACY.get(mode, mode)
    if mode not in P_SCALE_MODES:
        raise ValueError(f"NVFP4_P_SCALE_MODE must be one of {sorted(P_SCALE_MODES)}, got {mode!r}")
    divisors = P_SCALE_MODES[mode]
    divisor = divisors[0] if len(divisors) == 1 else 6.0
    if divisor_text is not None and float(divisor_text) != divisor:
        raise ValueError(f"NVFP4_P_SCALE_MODE={mode!r} contradicts NVFP4_P_SCALE_DIVISOR={divisor_text!r}")
    return mode, divisor, mode == "e2m1_max_grid"
