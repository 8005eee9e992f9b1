"""What sits between ``fp4_decode`` and the two launches of a decode call.

The public contract is the one of src/nvfp4_decode_kernel/_kernel.py of OpenBitSys/BitDecoding-FP4
(BF16 query or pre-quantized query, never both; a BF16 query may bring scratch, a scale mode, a
rotation and a tail write, a pre-quantized one may not; ``num_splits > 1`` is served or refused,
never quietly run as one tile). The organisation is this package's own: the call is reduced to a
:class:`QueryOperands` record by one of two resolvers and then handed to the unsplit or the split
launcher of ``_decode``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

import bdfp4

from .interface import RESIDUAL_ROW_TILE, DecodeTailWrite
from .scale_mode import DEFAULT_SCALE_MODE, scale_format, sf_vec_size

bdfp4.library()  # fail at import, loudly, when libbdfp4.so has not been built

HEAD_DIM = 128


@dataclass
class QueryOperands:
    """The FP4 query terms the decode kernel reads, the BF16 copy the tail and sink blocks read,
    and the softmax scale that goes with them."""

    fp4: torch.Tensor
    scales: torch.Tensor
    fp4_second: torch.Tensor | None
    scales_second: torch.Tensor | None
    padded_bf16: torch.Tensor | None
    softmax_scale: float


def _scratch_or_none(buffer, name: str, dtype, rows: int, inner: tuple, device):
    """A caller buffer must be contiguous, of the right element type and inner shape, and hold at
    least ``rows`` leading entries; ``None`` passes through."""
    if buffer is None:
        return None
    fits = (
        buffer.dtype is dtype and buffer.device == device and buffer.is_contiguous()
        and buffer.ndim == len(inner) + 1 and buffer.shape[0] >= rows and tuple(buffer.shape[1:]) == inner
    )
    if not fits:
        kind = "BF16" if dtype is torch.bfloat16 else "UINT8"
        raise ValueError(f"{name} must be contiguous {kind} [at least {rows}, {', '.join(map(str, inner))}]")
    return buffer


def _quantize_bf16_query(query, *, row_indices, heads_kv, needs_padded, terms, scale_mode, rotation, tail_write,
                         softmax_scale, scratch, tensor_scale) -> QueryOperands:
    """Run the query quantizer (and its fused tail write) into fresh or caller-owned buffers."""
    from ._quantize import quantize_query

    rows = query.shape[0] if row_indices is None else row_indices.shape[0]
    heads, dim = query.shape[1], query.shape[2]
    device = query.device
    atoms = dim // (4 * sf_vec_size(scale_mode))
    code_shape, scale_shape = (1, heads, dim // 2), (1, heads, atoms, 32, 4, 4)
    if terms == 1 and (scratch["fp4_second"] is not None or scratch["scales_second"] is not None):
        raise ValueError("second query scratch requires query_terms=2")
    owned = {
        "fp4": _scratch_or_none(scratch["fp4"], "query_fp4_scratch", torch.uint8, rows, code_shape, device),
        "scales": _scratch_or_none(scratch["scales"], "query_scales_scratch", torch.uint8, rows, scale_shape, device),
        "fp4_second": _scratch_or_none(scratch["fp4_second"], "query_fp4_second_scratch", torch.uint8, rows,
                                       code_shape, device),
        "scales_second": _scratch_or_none(scratch["scales_second"], "query_scales_second_scratch", torch.uint8, rows,
                                          scale_shape, device),
    }
    padded = None
    if needs_padded:
        # only row 0 of each 128-row tile is written per call; a caller's buffer was zeroed once by its owner
        tile = (RESIDUAL_ROW_TILE, heads, dim)
        given = _scratch_or_none(scratch["padded"], "query_padded_scratch", torch.bfloat16, rows, tile, device)
        padded = given[:rows] if given is not None else torch.zeros((rows, *tile), dtype=torch.bfloat16, device=device)
    result = quantize_query(
        query, row_indices=row_indices, query_padded_out=padded, heads_kv=heads_kv,
        query_fp4_scratch=owned["fp4"], query_scales_scratch=owned["scales"],
        query_fp4_second_scratch=owned["fp4_second"], query_scales_second_scratch=owned["scales_second"],
        query_terms=terms, scale_mode=scale_mode, rotation=rotation, tail_write=tail_write,
        tensor_scale=tensor_scale,
    )
    second = result[2:] if terms == 2 else (None, None)
    return QueryOperands(result[0], result[1], second[0], second[1], padded,
                         dim ** -0.5 if softmax_scale is None else softmax_scale)


def _accept_quantized_query(fp4, scales, fp4_second, scales_second, *, terms, softmax_scale,
                            bf16_only: dict) -> QueryOperands:
    """A query quantized by the caller is taken as it is; whatever configures the quantizer has no
    meaning then and is refused rather than ignored."""
    if fp4 is None or scales is None:
        raise ValueError("query_fp4 and query_scales must be provided together")
    if (fp4_second is None) != (scales_second is None):
        raise ValueError("query_fp4_second and query_scales_second must be provided together")
    if terms == 2 and fp4_second is None:
        raise ValueError("query_terms=2 needs query_fp4_second and query_scales_second")
    if terms == 1 and fp4_second is not None:
        raise ValueError("second pre-quantized query pair requires query_terms=2")
    stray = [name for name, (value, neutral) in bf16_only.items()
             if not (value is neutral or (isinstance(neutral, str) and value == neutral))]
    if stray:
        raise ValueError(f"{stray[0]} applies only to the BF16 query path")
    return QueryOperands(fp4, scales, fp4_second, scales_second, None,
                         HEAD_DIM ** -0.5 if softmax_scale is None else softmax_scale)


def fp4_decode_impl(
    query, key_pages_fp4, key_scales, value_pages_fp4, value_scales, fp4_page_table, seqused_fp4, *,
    query_fp4=None, query_scales=None, query_fp4_second=None, query_scales_second=None,
    residual_key_pages_bf16=None, residual_value_pages_bf16=None, residual_page_ids=None,
    seqused_residual=None, seqused_sink=None, has_bf16=None, softmax_scale=None, query_row_indices=None,
    out=None, out_indices=None, trusted_metadata=False, num_splits=1, query_padded_scratch=None,
    query_fp4_scratch=None, query_scales_scratch=None, query_fp4_second_scratch=None,
    query_scales_second_scratch=None, split_partial_scratch=None, split_lse_scratch=None, query_terms=1,
    scale_mode=DEFAULT_SCALE_MODE, query_rotation="none", tail_write: DecodeTailWrite | None = None,
    split_merge_counters=None, row_order=None, tensor_scales=None, row_splits=None,
):
    from ._decode import decode_fp4, decode_fp4_split

    if isinstance(num_splits, bool) or not isinstance(num_splits, int) or num_splits < 1:
        raise ValueError(f"num_splits must be a positive integer, got {num_splits!r}")
    if query_terms not in (1, 2):
        raise ValueError(f"query_terms must be 1 or 2, got {query_terms!r}")
    fmt = scale_format(scale_mode)
    key_ts, query_ts, value_ts = (1.0, 1.0, 1.0) if tensor_scales is None else map(float, tensor_scales)
    given_fp4 = any(t is not None for t in (query_fp4, query_scales, query_fp4_second, query_scales_second))
    if (query is None) == (not given_fp4):
        raise ValueError("supply either BF16 query or query_fp4 + query_scales")

    residual = (residual_key_pages_bf16, residual_value_pages_bf16, residual_page_ids, seqused_residual)
    if query is not None:
        operands = _quantize_bf16_query(
            query, row_indices=query_row_indices, heads_kv=key_pages_fp4.shape[2],
            needs_padded=residual_key_pages_bf16 is not None, terms=query_terms, scale_mode=scale_mode,
            rotation=query_rotation, tail_write=tail_write, softmax_scale=softmax_scale, tensor_scale=query_ts,
            scratch={"padded": query_padded_scratch, "fp4": query_fp4_scratch, "scales": query_scales_scratch,
                     "fp4_second": query_fp4_second_scratch, "scales_second": query_scales_second_scratch})
    else:
        operands = _accept_quantized_query(
            query_fp4, query_scales, query_fp4_second, query_scales_second, terms=query_terms,
            softmax_scale=softmax_scale,
            bf16_only={"query_row_indices": (query_row_indices, None), "query_padded_scratch": (query_padded_scratch, None),
                       "query_fp4_scratch": (query_fp4_scratch, None), "query_scales_scratch": (query_scales_scratch, None),
                       "query_fp4_second_scratch": (query_fp4_second_scratch, None),
                       "query_scales_second_scratch": (query_scales_second_scratch, None),
                       "scale_mode": (scale_mode, DEFAULT_SCALE_MODE), "query_rotation": (query_rotation, "none"),
                       "tail_write": (tail_write, None)})

    if num_splits > 1:
        # the split path merges the BF16 blocks inside one of its parts, which needs all of them and the
        # BF16 query copy; with no residual at all there is nothing to merge
        bare = all(arg is None for arg in residual) and has_bf16 is None
        whole = all(arg is not None for arg in residual) and operands.padded_bf16 is not None
        if not (bare or whole):
            raise ValueError(
                "num_splits > 1 needs either no residual argument at all or a complete residual on the BF16 "
                "query path; this combination runs on the single-tile path only")
        if out_indices is not None:
            raise ValueError("num_splits > 1 cannot be combined with out_indices: the merge writes rows in order")

    common = dict(
        query_fp4=operands.fp4, query_scales=operands.scales, query_fp4_second=operands.fp4_second,
        query_scales_second=operands.scales_second, query_padded_bf16=operands.padded_bf16,
        key_pages_fp4=key_pages_fp4, key_scales=key_scales, value_pages_fp4=value_pages_fp4,
        value_scales=value_scales, fp4_page_table=fp4_page_table, seqused_fp4=seqused_fp4,
        residual_key_pages_bf16=residual_key_pages_bf16, residual_value_pages_bf16=residual_value_pages_bf16,
        residual_page_ids=residual_page_ids, seqused_residual=seqused_residual, seqused_sink=seqused_sink,
        has_bf16=has_bf16, softmax_scale=operands.softmax_scale, out=out, scale_format=fmt, row_order=row_order,
        tensor_scales=(key_ts, query_ts, value_ts),
    )
    if num_splits == 1:
        return decode_fp4(**common, out_indices=out_indices, trusted_metadata=trusted_metadata)
    decode_fp4(**common, out_indices=out_indices, trusted_metadata=trusted_metadata, validate_only=True)
    return decode_fp4_split(
        **common, num_splits=num_splits, split_partial_scratch=split_partial_scratch,
        split_lse_scratch=split_lse_scratch, split_merge_counters=split_merge_counters, row_splits=row_splits)
