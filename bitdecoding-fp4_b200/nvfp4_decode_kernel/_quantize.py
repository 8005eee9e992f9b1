"""NVFP4 query quantization with caller-suppliable scratch.

``quantize_query`` keeps the signature and return convention of
src/nvfp4_decode_kernel/_quantize.py:16-205 of OpenBitSys/BitDecoding-FP4.
"""

from __future__ import annotations

import torch

from .interface import DecodeTailWrite
from .quantize_kv_kernel import quantize_key_pages, quantize_value_pages  # noqa: F401  (re-exported)
from .quantize_q_kernel import quantize_decode_q_to_padded_fp4
from .scale_mode import DEFAULT_SCALE_MODE, sf_vec_size

PAGE_SIZE = 128


def _scale_view(storage: torch.Tensor, heads_kv: int) -> torch.Tensor:
    """Storage ``[rows,1,Hq,rest_k,32,4,4]`` u8 -> the ``(32,4,1,4,rest_k,heads_kv,rows)`` view the
    decode kernel validates: head slot ``k`` of a row holds the scale tile of KV head ``k``."""
    rows, _, heads, rest_k = storage.shape[:4]
    s = storage.stride()
    return storage.as_strided(
        (32, 4, 1, 4, rest_k, heads_kv, rows),
        (s[4], s[5], s[1], s[6], s[3], s[2], s[0]),
        storage.storage_offset(),
    )


def quantize_query(
    query: torch.Tensor,
    *,
    row_indices: torch.Tensor | None = None,
    query_padded_out: torch.Tensor | None = None,
    heads_kv: int | None = None,
    query_fp4_scratch: torch.Tensor | None = None,
    query_scales_scratch: torch.Tensor | None = None,
    query_fp4_second_scratch: torch.Tensor | None = None,
    query_scales_second_scratch: torch.Tensor | None = None,
    query_terms: int = 1,
    scale_mode: str = DEFAULT_SCALE_MODE,
    rotation: str = "none",
    tail_write: DecodeTailWrite | None = None,
    tensor_scale: float = 1.0,
):
    """Quantize BF16 decode rows; returns ``(q, s)`` or, with two terms, ``(q0, s0, q1, s1)``.

    Outputs may come from the caller and may be wider than this batch; a supplied scale buffer
    must arrive zeroed, because only the ``heads // heads_kv`` scale rows of each KV-head tile
    that carry a query head are ever written, and it belongs to one ``(heads, heads_kv,
    head_dim)`` geometry for its whole life. ``tensor_scale`` (no reference counterpart) is an FP32
    per-tensor scale: the terms then hold ``query / tensor_scale``.
    """
    if query_terms not in (1, 2):
        raise ValueError(f"query_terms must be 1 or 2, got {query_terms!r}")
    if query_terms == 1 and (query_fp4_second_scratch is not None or query_scales_second_scratch is not None):
        raise ValueError("second query scratch requires query_terms=2")
    if query.dtype is not torch.bfloat16 or not query.is_cuda:
        raise ValueError("query must be a BF16 CUDA tensor")
    if query.ndim != 3 or query.stride(-1) != 1:
        raise ValueError("query must have shape [rows, heads, head_dim]")
    if row_indices is not None and (
        row_indices.dtype is not torch.int32
        or not row_indices.is_cuda
        or not row_indices.is_contiguous()
        or row_indices.ndim != 1
    ):
        raise ValueError("row_indices must be contiguous 1-D INT32 CUDA")
    _, heads, head_dim = query.shape
    heads_kv = heads if heads_kv is None else heads_kv
    if heads_kv < 1 or heads % heads_kv:
        raise ValueError("query heads must be divisible by heads_kv")
    rows = query.shape[0] if row_indices is None else row_indices.shape[0]
    atom_k = 4 * sf_vec_size(scale_mode)
    if head_dim % atom_k:
        raise ValueError(f"query head_dim must be divisible by {atom_k}")
    rest_k = head_dim // atom_k

    def term_buffers(fp4_scratch, scales_scratch):
        fp4 = (
            torch.zeros(rows, 1, heads, head_dim // 2, dtype=torch.uint8, device=query.device)
            if fp4_scratch is None else fp4_scratch[:rows]
        ).view(torch.float4_e2m1fn_x2)
        storage = (
            torch.zeros(rows, 1, heads, rest_k, 32, 4, 4, dtype=torch.uint8, device=query.device)
            if scales_scratch is None else scales_scratch[:rows]
        )
        return fp4, _scale_view(storage, heads_kv)

    query_fp4, query_scales = term_buffers(query_fp4_scratch, query_scales_scratch)
    second = (None, None)
    if query_terms == 2:
        second = term_buffers(query_fp4_second_scratch, query_scales_second_scratch)
    quantize_decode_q_to_padded_fp4(
        query, query_fp4, query_scales, query_padded_out,
        query_fp4_out_2=second[0], query_scales_out_2=second[1],
        row_indices=row_indices, heads_kv=heads_kv, scale_mode=scale_mode, rotation=rotation,
        tail_write=tail_write, tensor_scale=tensor_scale,
    )
    if query_terms == 2:
        return query_fp4, query_scales, second[0], second[1]
    return query_fp4, query_scales
