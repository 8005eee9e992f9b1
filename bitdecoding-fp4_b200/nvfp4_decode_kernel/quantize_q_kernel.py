"""Decode-query quantization, backed by ``bdfp4_quantize_query``.

``quantize_decode_q_to_padded_fp4`` keeps the signature and argument contract of
src/nvfp4_decode_kernel/quantize_q_kernel.py:681-1110 of OpenBitSys/BitDecoding-FP4.
"""

from __future__ import annotations

from typing import Optional

import torch

import bdfp4

from .interface import DecodeTailWrite
from .scale_mode import DEFAULT_SCALE_MODE, mode_id, sf_vec_size

PAGE_SIZE = 128
SF_VEC_SIZE = 16
GROUPS_PER_ATOM = 4
QUERY_ROTATIONS = ("none", "hadamard")


def _check_tail_write(tail: DecodeTailWrite, rows: int, heads_kv: int, head_dim: int, device) -> None:
    expected_tail = (PAGE_SIZE + tail.sink_tokens, heads_kv, head_dim)
    for name in ("key", "value"):
        tensor = getattr(tail, name)
        if (
            tensor.dtype is not torch.bfloat16
            or tensor.device != device
            or tensor.ndim != 3
            or tensor.shape[0] < rows
            or tuple(tensor.shape[1:]) != (heads_kv, head_dim)
            or tensor.stride()[1:] != (head_dim, 1)
            or tensor.stride(0) % 8
            or tensor.data_ptr() % 16
        ):
            raise ValueError(f"tail_write.{name} must be BF16 [>= rows, heads_kv, head_dim], dense within a token")
    for name in ("tail_key", "tail_value"):
        tensor = getattr(tail, name)
        if (
            tensor.dtype is not torch.bfloat16
            or tensor.device != device
            or tensor.ndim != 4
            or tuple(tensor.shape[1:]) != expected_tail
            or tensor.stride()[1:] != (heads_kv * head_dim, head_dim, 1)
        ):
            raise ValueError(
                f"tail_write.{name} must be BF16 [slots, {expected_tail[0]}, heads_kv, head_dim], dense within a slot"
            )
    for name in ("row_to_slot", "seq_lens", "seqused_fp4"):
        tensor = getattr(tail, name)
        if (
            tensor.dtype is not torch.int32
            or tensor.device != device
            or not tensor.is_contiguous()
            or tensor.ndim != 1
            or tensor.shape[0] < rows
        ):
            raise ValueError(f"tail_write.{name} must be contiguous INT32 with at least one entry per row")
    if tail.key_shift is not None and (
        tail.key_shift.dtype is not torch.float32
        or tail.key_shift.device != device
        or not tail.key_shift.is_contiguous()
        or tuple(tail.key_shift.shape) != (heads_kv, head_dim)
    ):
        raise ValueError("tail_write.key_shift must be contiguous FP32 [heads_kv, head_dim]")
    if not 0 <= tail.sink_tokens <= 16:
        raise ValueError("tail_write.sink_tokens must lie in [0, 16]")


def quantize_decode_q_to_padded_fp4(
    query: torch.Tensor,
    query_fp4_out: torch.Tensor,
    query_scales_out: torch.Tensor,
    query_padded_out: Optional[torch.Tensor] = None,
    *,
    query_fp4_out_2: Optional[torch.Tensor] = None,
    query_scales_out_2: Optional[torch.Tensor] = None,
    row_indices: Optional[torch.Tensor] = None,
    heads_kv: Optional[int] = None,
    scale_mode: str = DEFAULT_SCALE_MODE,
    rotation: str = "none",
    tail_write: Optional[DecodeTailWrite] = None,
    tensor_scale: float = 1.0,
) -> None:
    """Quantize selected BF16 query rows into preallocated outputs.

    ``rotation="hadamard"`` first multiplies each head by the normalized Sylvester Hadamard in
    FP32; both terms are quantized from those FP32 values and the padded copy holds them rounded
    to BF16. ``tail_write`` also places each row's new K/V token in the BF16 tail from extra CTAs
    of the same launch.
    """
    if not (tensor_scale > 0.0 and tensor_scale < float("inf")):
        raise ValueError("tensor_scale must be finite and positive")
    if rotation not in QUERY_ROTATIONS:
        raise ValueError(f"rotation must be one of {QUERY_ROTATIONS}, got {rotation!r}")
    if query.dtype is not torch.bfloat16 or not query.is_cuda:
        raise ValueError("query must be a BF16 CUDA tensor")
    if query.ndim != 3 or query.stride(-1) != 1:
        raise ValueError("query must have shape [rows, heads, head_dim]")
    if query.data_ptr() % 16 or query.stride(0) % 8 or query.stride(1) % 8:
        raise ValueError(
            "every query head vector must start on a 16-byte boundary: "
            "the data pointer must be 16-byte aligned and the row and head "
            "strides multiples of 8 elements"
        )
    source_rows, heads, head_dim = query.shape
    if head_dim != 128:
        raise ValueError("query head_dim must be 128")
    heads_kv = heads if heads_kv is None else heads_kv
    if heads_kv < 1 or heads % heads_kv:
        raise ValueError("query heads must be divisible by heads_kv")
    rows = query_fp4_out.shape[0]
    if row_indices is None:
        if source_rows != rows:
            raise ValueError("query rows must match output rows")
    elif (
        row_indices.dtype is not torch.int32
        or not row_indices.is_cuda
        or row_indices.device != query.device
        or not row_indices.is_contiguous()
        or row_indices.shape != (rows,)
    ):
        raise ValueError("row_indices must be contiguous INT32 CUDA with shape [rows]")

    rest_k = head_dim // (GROUPS_PER_ATOM * sf_vec_size(scale_mode))  # scale atoms per head: 2 (NVFP4) or 1 (MXFP4)
    expected_fp4_shape = (rows, 1, heads, head_dim // 2)
    expected_scales_shape = (32, 4, 1, 4, rest_k, heads_kv, rows)
    expected_scales_strides = (16, 4, heads * rest_k * 512, 1, 512, rest_k * 512, heads * rest_k * 512)
    if (query_fp4_out_2 is None) != (query_scales_out_2 is None):
        raise ValueError("query_fp4_out_2 and query_scales_out_2 must be provided together")
    fp4_dtypes = (torch.float4_e2m1fn_x2, torch.uint8)

    def check_pair(fp4, scales, suffix):
        if (
            tuple(fp4.shape) != expected_fp4_shape
            or fp4.dtype not in fp4_dtypes
            or not fp4.is_cuda
            or fp4.device != query.device
            or not fp4.is_contiguous()
        ):
            raise ValueError(f"query_fp4_out{suffix} must have shape {expected_fp4_shape}")
        if (
            tuple(scales.shape) != expected_scales_shape
            or scales.dtype is not torch.uint8
            or not scales.is_cuda
            or scales.device != query.device
        ):
            raise ValueError(f"query_scales_out{suffix} must have shape {expected_scales_shape}")
        if rows > 0 and scales.stride() != expected_scales_strides:
            raise ValueError(f"query_scales_out{suffix} must use the layout returned by quantize_query")

    check_pair(query_fp4_out, query_scales_out, "")
    if query_fp4_out_2 is not None:
        check_pair(query_fp4_out_2, query_scales_out_2, "_2")
    if query_padded_out is not None and (
        query_padded_out.dtype is not torch.bfloat16
        or query_padded_out.device != query.device
        or tuple(query_padded_out.shape) != (rows, PAGE_SIZE, heads, head_dim)
        or not query_padded_out.is_contiguous()
    ):
        raise ValueError(
            f"query_padded_out must be contiguous BF16 with shape {(rows, PAGE_SIZE, heads, head_dim)}"
        )
    if tail_write is not None:
        _check_tail_write(tail_write, rows, heads_kv, head_dim, query.device)
    if rows == 0:
        return

    a = bdfp4.QuantizeQueryArgs()
    a.query = query.data_ptr()
    a.query_row_stride, a.query_head_stride = query.stride(0), query.stride(1)
    a.row_indices = bdfp4.ptr(row_indices)
    a.rows, a.heads_q, a.heads_kv = rows, heads, heads_kv
    a.scale_mode = mode_id(scale_mode)
    a.tensor_scale = float(tensor_scale)
    a.rotate = int(rotation == "hadamard")
    a.query_codes, a.query_scales = query_fp4_out.data_ptr(), query_scales_out.data_ptr()
    a.query_codes_second, a.query_scales_second = bdfp4.ptr(query_fp4_out_2), bdfp4.ptr(query_scales_out_2)
    a.query_padded = bdfp4.ptr(query_padded_out)
    if tail_write is not None:
        t = tail_write
        a.new_key, a.new_value = t.key.data_ptr(), t.value.data_ptr()
        a.new_key_token_pitch, a.new_value_token_pitch = t.key.stride(0), t.value.stride(0)
        a.tail_key, a.tail_value = t.tail_key.data_ptr(), t.tail_value.data_ptr()
        a.tail_slot_stride = t.tail_key.stride(0)
        a.row_to_slot, a.seq_lens, a.seqused_fp4 = t.row_to_slot.data_ptr(), t.seq_lens.data_ptr(), t.seqused_fp4.data_ptr()
        a.rotate_key = int(bool(t.rotate_key))
        a.key_shift = bdfp4.ptr(t.key_shift)
        a.sink_tokens = int(t.sink_tokens)
    bdfp4.quantize_query(a, bdfp4.current_stream(query.device))
