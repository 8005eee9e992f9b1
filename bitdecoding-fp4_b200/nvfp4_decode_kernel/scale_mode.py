"""Names of the block-scale rules the quantizers accept.

An NVFP4 mode is a tuple of divisors: a group of sixteen values stores
``E4M3(amax / d)`` for whichever ``d`` reconstructs it with the least squared error, the
earliest divisor winning ties, so ``amax6`` is the answer whenever nothing beats it and each
longer tuple only ever improves on its prefix. Mirrors
src/nvfp4_decode_kernel/scale_mode.py of OpenBitSys/BitDecoding-FP4 (same names and results).
The MXFP4 modes store one E8M0 power-of-two scale per 32 values, picked by an exponent rule.
"""

from __future__ import annotations

SCALE_MODES: dict[str, tuple[float, ...]] = {
    "amax6": (6.0,),
    "four_six": (6.0, 4.0),
    "four_six_sixhalf": (6.0, 4.0, 6.5),
}
DEFAULT_SCALE_MODE = "amax6"
MX_SCALE_MODES: dict[str, str] = {
    "mxfp4_ocp": "ocp",
    "mxfp4_round_up": "round_up",
    "mxfp4_search": "search",
}
_PER_TENSOR_FIELDS = ("key", "query", "value")


def candidates(scale_mode: str) -> tuple[float, ...]:
    """Divisors of an NVFP4 mode in tie-break order."""
    if scale_mode not in SCALE_MODES:
        known = sorted(SCALE_MODES) + sorted(MX_SCALE_MODES)
        raise ValueError(f"unknown scale_mode {scale_mode!r}, expected one of {known}")
    return SCALE_MODES[scale_mode]


def scale_format(scale_mode: str) -> str:
    """``"nvfp4"`` or ``"mxfp4"``."""
    if scale_mode in MX_SCALE_MODES:
        return "mxfp4"
    candidates(scale_mode)
    return "nvfp4"


def sf_vec_size(scale_mode: str) -> int:
    """Values sharing one scale: 16 for NVFP4, 32 for MXFP4."""
    return 16 if scale_format(scale_mode) == "nvfp4" else 32


def scale_rule(scale_mode: str):
    """The divisors of an NVFP4 mode, or the exponent rule name of an MX mode."""
    return MX_SCALE_MODES[scale_mode] if scale_mode in MX_SCALE_MODES else candidates(scale_mode)


def parse_scale_mode_spec(spec: str):
    """``"four_six"`` -> itself; ``"key=a,value=b,query=c"`` -> a dict with exactly those keys."""
    if "=" not in spec:
        return spec
    modes = {}
    for part in filter(None, spec.split(",")):
        name, _, mode = part.partition("=")
        modes[name] = mode
    if sorted(modes) != list(_PER_TENSOR_FIELDS):
        raise ValueError(
            f"a per-tensor scale mode needs exactly {list(_PER_TENSOR_FIELDS)}, got {sorted(modes)}"
        )
    return modes


def mode_id(scale_mode: str) -> int:
    """Integer the C ABI uses for a mode (``BDFP4_SCALE_*``): the NVFP4 candidate sets 0-2, then the
    MXFP4 rules 3-5."""
    if scale_format(scale_mode) == "mxfp4":
        return len(SCALE_MODES) + list(MX_SCALE_MODES).index(scale_mode)
    return list(SCALE_MODES).index(scale_mode)
