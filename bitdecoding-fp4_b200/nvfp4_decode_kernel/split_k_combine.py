"""LSE-weighted reduction of split-KV decode partials into the BF16 output.

``combine_split_partials`` keeps the signature of
src/nvfp4_decode_kernel/split_k_combine.py:86-133 of OpenBitSys/BitDecoding-FP4 and runs
``bdfp4_combine`` on torch's current stream (the stream the partials were written on).
"""

from __future__ import annotations

import torch

import bdfp4


def combine_split_partials(out_partial: torch.Tensor, lse_partial: torch.Tensor, out: torch.Tensor | None = None):
    """``out_partial`` ``(splits, rows, 1, heads, 128)`` FP32 under ``lse_partial``
    ``(splits, rows, 1, heads)`` FP32 -> BF16 ``(rows, 1, heads, 128)``, written to ``out`` when given."""
    num_splits, rows, seqlen, heads, head_dim = out_partial.shape
    if seqlen != 1:
        raise ValueError(f"the split-K combine serves one query position, got {seqlen}")
    if head_dim != 128:
        raise ValueError("the split-K combine serves head_dim 128")
    if out_partial.dtype is not torch.float32 or lse_partial.dtype is not torch.float32:
        raise ValueError("partials must be FP32")
    if not out_partial.is_contiguous() or not lse_partial.is_contiguous():
        raise ValueError("partials must be contiguous")
    if tuple(lse_partial.shape) != (num_splits, rows, 1, heads):
        raise ValueError("lse_partial must have shape (splits, rows, 1, heads)")
    if out is None:
        out = torch.empty(rows, seqlen, heads, head_dim, dtype=torch.bfloat16, device=out_partial.device)
    elif out.dtype is not torch.bfloat16 or out.stride(-1) != 1 or out.stride(-2) != head_dim:
        raise ValueError("out must be BF16, dense within a row")
    bdfp4.combine(out_partial, lse_partial, num_splits, rows, heads, out, out.stride(0),
                  bdfp4.current_stream(out_partial.device))
    return out
