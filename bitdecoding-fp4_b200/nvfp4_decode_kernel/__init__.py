"""Paged NVFP4 decode attention and KV quantize-on-write for B200 (sm_100a).

Drop-in for the ``nvfp4_decode_kernel`` package of OpenBitSys/BitDecoding-FP4: the same public
names (src/nvfp4_decode_kernel/__init__.py:7-21), served by hand-written CUDA kernels in
``libbdfp4.so``. Everything public lives in :mod:`.interface`; this file only re-exports it.
"""

from . import interface as _interface

__all__ = sorted(("fp4_decode", "DecodeTailWrite", "split_partial_count", "RESIDUAL_ROW_TILE",
                  "KernelNotAvailableError"))
globals().update({_name: getattr(_interface, _name) for _name in __all__})
SINK_TOKENS = _interface.SINK_TOKENS  # importable, but not part of ``__all__`` (as in the reference)
