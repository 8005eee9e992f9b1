"""The decode entry behind ``fp4_decode``: pick the query contract, quantize, dispatch.

Keeps the behaviour of src/nvfp4_decode_kernel/_kernel.py:93-416 of OpenBitSys/BitDecoding-FP4:
a BF16 query is quantized here (optionally into caller scratch, optionally with the fused tail
write); a pre-quantized query is taken as is; ``num_splits > 1`` is either served by the split
path or refused, never silently downgraded.
"""

from __future__ import annotations

import torch

import bdfp4

from .interface import RESIDUAL_ROW_TILE, DecodeTailWrite
from .scale_mode import DEFAULT_SCALE_MODE, scale_format, sf_vec_size

bdfp4.library()  # fail at import, loudly, when libbdfp4.so has not been built


def _padded_query_buffer(query: torch.Tensor, rows: int, scratch: torch.Tensor | None) -> torch.Tensor:
    """``[rows, 128, heads, dim]`` BF16 whose row 0 of each tile the quantizer fills. A caller's
    buffer is trusted to have been zeroed once; a fresh one is zeroed here."""
    shape = (rows, RESIDUAL_ROW_TILE, query.shape[1], query.shape[2])
    if scratch is None:
        return torch.zeros(shape, dtype=torch.bfloat16, device=query.device)
    if (
        scratch.dtype is not torch.bfloat16
        or scratch.device != query.device
        or scratch.ndim != 4
        or scratch.shape[0] < rows
        or tuple(scratch.shape[1:]) != shape[1:]
        or not scratch.is_contiguous()
    ):
        raise ValueError(
            f"query_padded_scratch must be contiguous BF16 [at least {rows}, {shape[1]}, {shape[2]}, {shape[3]}]"
        )
    return scratch[:rows]


def _check_quantizer_scratch(scratch, name: str, rows: int, inner: tuple, device) -> None:
    if scratch is None:
        return
    if (
        scratch.dtype is not torch.uint8
        or scratch.device != device
        or scratch.shape[0] < rows
        or tuple(scratch.shape[1:]) != inner
        or not scratch.is_contiguous()
    ):
        raise ValueError(f"{name} must be contiguous UINT8 [at least {rows}, {', '.join(map(str, inner))}]")


def fp4_decode_impl(
    query, key_pages_fp4, key_scales, value_pages_fp4, value_scales, fp4_page_table, seqused_fp4, *,
    query_fp4=None, query_scales=None, query_fp4_second=None, query_scales_second=None,
    residual_key_pages_bf16=None, residual_value_pages_bf16=None, residual_page_ids=None,
    seqused_residual=None, seqused_sink=None, has_bf16=None, softmax_scale=None, query_row_indices=None,
    out=None, out_indices=None, trusted_metadata=False, num_splits=1, query_padded_scratch=None,
    query_fp4_scratch=None, query_scales_scratch=None, query_fp4_second_scratch=None,
    query_scales_second_scratch=None, split_partial_scratch=None, split_lse_scratch=None, query_terms=1,
    scale_mode=DEFAULT_SCALE_MODE, query_rotation="none", tail_write: DecodeTailWrite | None = None,
    split_merge_counters=None, row_order=None,
):
    from ._decode import decode_fp4, decode_fp4_split
    from ._quantize import quantize_query

    if not isinstance(num_splits, int) or isinstance(num_splits, bool) or num_splits < 1:
        raise ValueError(f"num_splits must be a positive integer, got {num_splits!r}")
    if query_terms not in (1, 2):
        raise ValueError(f"query_terms must be 1 or 2, got {query_terms!r}")
    fmt = scale_format(scale_mode)
    prequantized = (query_fp4, query_scales, query_fp4_second, query_scales_second)
    has_fp4_query = any(t is not None for t in prequantized)
    if (query is not None) == has_fp4_query:
        raise ValueError("supply either BF16 query or query_fp4 + query_scales")

    query_padded_bf16 = None
    if query is not None:
        if softmax_scale is None:
            softmax_scale = query.shape[-1] ** -0.5
        rows = query.shape[0] if query_row_indices is None else query_row_indices.shape[0]
        if residual_key_pages_bf16 is not None:
            query_padded_bf16 = _padded_query_buffer(query, rows, query_padded_scratch)
        heads, head_dim = query.shape[1], query.shape[2]
        sf_inner = (1, heads, head_dim // (4 * sf_vec_size(scale_mode)), 32, 4, 4)
        _check_quantizer_scratch(query_fp4_scratch, "query_fp4_scratch", rows, (1, heads, head_dim // 2), query.device)
        _check_quantizer_scratch(query_scales_scratch, "query_scales_scratch", rows, sf_inner, query.device)
        if query_terms == 1 and (query_fp4_second_scratch is not None or query_scales_second_scratch is not None):
            raise ValueError("second query scratch requires query_terms=2")
        if query_terms == 2:
            _check_quantizer_scratch(
                query_fp4_second_scratch, "query_fp4_second_scratch", rows, (1, heads, head_dim // 2), query.device
            )
            _check_quantizer_scratch(
                query_scales_second_scratch, "query_scales_second_scratch", rows, sf_inner, query.device
            )
        quantized = quantize_query(
            query, row_indices=query_row_indices, query_padded_out=query_padded_bf16,
            heads_kv=key_pages_fp4.shape[2], query_fp4_scratch=query_fp4_scratch,
            query_scales_scratch=query_scales_scratch, query_fp4_second_scratch=query_fp4_second_scratch,
            query_scales_second_scratch=query_scales_second_scratch, query_terms=query_terms,
            scale_mode=scale_mode, rotation=query_rotation, tail_write=tail_write,
        )
        query_fp4, query_scales = quantized[0], quantized[1]
        query_fp4_second, query_scales_second = (quantized[2], quantized[3]) if query_terms == 2 else (None, None)
    else:
        if query_fp4 is None or query_scales is None:
            raise ValueError("query_fp4 and query_scales must be provided together")
        if (query_fp4_second is None) != (query_scales_second is None):
            raise ValueError("query_fp4_second and query_scales_second must be provided together")
        has_second = query_fp4_second is not None
        if query_terms == 2 and not has_second:
            raise ValueError("query_terms=2 needs query_fp4_second and query_scales_second")
        if query_terms == 1 and has_second:
            raise ValueError("second pre-quantized query pair requires query_terms=2")
        if query_row_indices is not None:
            raise ValueError("query_row_indices applies only to the BF16 query path")
        for name, scratch in (
            ("query_padded_scratch", query_padded_scratch), ("query_fp4_scratch", query_fp4_scratch),
            ("query_scales_scratch", query_scales_scratch),
            ("query_fp4_second_scratch", query_fp4_second_scratch),
            ("query_scales_second_scratch", query_scales_second_scratch),
        ):
            if scratch is not None:
                raise ValueError(f"{name} applies only to the BF16 query path")
        if scale_mode != DEFAULT_SCALE_MODE:
            raise ValueError("scale_mode applies only to the BF16 query path")
        if query_rotation != "none":
            raise ValueError("query_rotation applies only to the BF16 query path")
        if tail_write is not None:
            raise ValueError("tail_write applies only to the BF16 query path")
        if softmax_scale is None:
            softmax_scale = 128 ** -0.5

    residual = (residual_key_pages_bf16, residual_value_pages_bf16, residual_page_ids, seqused_residual)
    complete_residual = all(arg is not None for arg in residual)
    splittable = (all(arg is None for arg in residual) and has_bf16 is None) or (
        complete_residual and query_padded_bf16 is not None
    )
    if num_splits > 1 and not splittable:
        raise ValueError(
            "num_splits > 1 needs either no residual argument at all or a "
            "complete residual on the BF16 query path; this combination "
            "runs on the single-tile path only"
        )
    if num_splits > 1 and out_indices is not None:
        raise ValueError(
            "num_splits > 1 cannot be combined with out_indices, because the "
            "split path's combine writes the batch's rows in order"
        )
    common = dict(
        query_fp4=query_fp4, query_scales=query_scales, query_fp4_second=query_fp4_second,
        query_scales_second=query_scales_second, query_padded_bf16=query_padded_bf16,
        key_pages_fp4=key_pages_fp4, key_scales=key_scales, value_pages_fp4=value_pages_fp4,
        value_scales=value_scales, fp4_page_table=fp4_page_table, seqused_fp4=seqused_fp4,
        residual_key_pages_bf16=residual_key_pages_bf16, residual_value_pages_bf16=residual_value_pages_bf16,
        residual_page_ids=residual_page_ids, seqused_residual=seqused_residual, seqused_sink=seqused_sink,
        has_bf16=has_bf16, softmax_scale=softmax_scale, out=out, scale_format=fmt, row_order=row_order,
    )
    if num_splits > 1:
        decode_fp4(**common, out_indices=out_indices, trusted_metadata=trusted_metadata, validate_only=True)
        return decode_fp4_split(
            **common, num_splits=num_splits, split_partial_scratch=split_partial_scratch,
            split_lse_scratch=split_lse_scratch, split_merge_counters=split_merge_counters,
        )
    return decode_fp4(**common, out_indices=out_indices, trusted_metadata=trusted_metadata)
