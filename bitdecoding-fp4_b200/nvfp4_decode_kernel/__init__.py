"""Paged NVFP4 decode attention and KV quantize-on-write for B200 (sm_100a).

Drop-in for the ``nvfp4_decode_kernel`` package of OpenBitSys/BitDecoding-FP4: the same public
names (src/nvfp4_decode_kernel/__init__.py:7-21), served by hand-written CUDA kernels in
``libbdfp4.so``.
"""

from .interface import (
    RESIDUAL_ROW_TILE,
    SINK_TOKENS,
    DecodeTailWrite,
    KernelNotAvailableError,
    fp4_decode,
    split_partial_count,
)

__all__ = [
    "RESIDUAL_ROW_TILE",
    "DecodeTailWrite",
    "KernelNotAvailableError",
    "fp4_decode",
    "split_partial_count",
]
