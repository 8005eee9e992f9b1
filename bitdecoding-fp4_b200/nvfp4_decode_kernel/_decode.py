"""Host dispatch of the paged FP4 decode kernel: validation, scratch contracts, launch.

``decode_fp4``, ``decode_fp4_split`` and ``split_k_heuristic`` keep the contracts of
src/nvfp4_decode_kernel/_decode.py (:697-1241, :1244-1456, :54-112) of OpenBitSys/BitDecoding-FP4.
The kernels are prebuilt in ``libbdfp4.so``, so there is no compile cache; the probability
scale rule and its threshold are launch arguments read from the environment per call.
"""

from __future__ import annotations

import functools
import math

import torch

import bdfp4

from .interface import SINK_TOKENS, split_partial_count
from .p_scale import BUILT_P_SCALE_MODES, resolve_p_scale_environment, resolve_p_scale_tau

PAGE_SIZE = 128
# values per scale: NVFP4 stores an E4M3 scale per 16, MXFP4 an E8M0 scale per 32
SCALE_FORMATS = {"nvfp4": 16, "mxfp4": 32}
# Cache page sizes this build serves. 128 is the reference's only size; with 64-token pages (no
# reference counterpart) a sequence still moves to FP4 in 128-token steps, two page-table entries
# each, and the page size is read off the shape of ``key_pages_fp4``.
CACHE_PAGE_SIZES = (128, 64)
HEAD_DIM = 128
SM100_MAJOR = 10
MAX_QUERY_HEADS_PER_KV_HEAD = 16
# Pages the split that also merges the BF16 tail and sink is charged for them (the reference's even
# partition is 0). Measured on B200 with one KV head per GPU (64 rows x 9 splits, every CTA resident at
# once, so the split that carries the two blocks ends last): 0 -> 131.5-133.1 us per step, 5 -> 129.9,
# 9 -> 128.0-128.6, 14 -> 131.2. With few long splits per row the charge is lost in the noise.
BF16_BLOCK_PAGE_COST = 8


def split_k_heuristic(rows: int, heads_kv: int, max_pages_per_row: int, *, sms: int) -> int:
    """Split count for a pure-FP4 decode by predicted makespan.

    A CTA walks one (row, KV head) pair's share of the pages, so a launch costs (scheduling
    rounds) x (pages per CTA + a pipeline fill of about 8 page times). Splitting divides the
    second factor and multiplies the first; a power-of-two count in 2..32 is taken only when it
    beats the unsplit makespan by more than the split path's own overhead (a factor 6/5), fewest
    splits first, and never below two pages per split. Uses the page table's width, not device
    lengths, so it costs no synchronisation.
    """
    if rows < 1 or heads_kv < 1 or max_pages_per_row < 2 or sms < 1:
        return 1
    ctas = rows * heads_kv
    fill = 8

    def makespan(splits: int) -> int:
        return math.ceil(ctas * splits / sms) * (math.ceil(max_pages_per_row / splits) + fill)

    best, best_cost = 1, None
    for splits in (2, 4, 8, 16, 32):
        if 2 * splits > max_pages_per_row:
            break
        cost = makespan(splits)
        if best_cost is None or cost < best_cost:
            best, best_cost = splits, cost
    if best_cost is None or 6 * best_cost >= 5 * makespan(1):
        return 1
    return best


def resident_num_splits(rows: int, heads_kv: int, *, sms: int, ctas_per_sm: int = 4, max_splits: int = 64) -> int:
    """Split count that keeps the whole launch resident at ``ctas_per_sm`` CTAs per SM.

    The decode kernel is bound by HBM only while enough independent CTAs stream at once: each CTA's
    per-page softmax chain has a fixed latency, and four CTAs per SM (what the two-stage kernel
    variant fits) hide it. With few (row, KV head) tiles (a small batch, or a KV-head slice of a
    tensor-parallel rank) this asks for more partitions than ``split_k_heuristic`` or the serving
    plugin's ``decode_num_splits`` would. Like them it uses the batch width only, never device
    lengths, so it is safe under CUDA-graph replay. Not part of the reference's API. (16 tiles of eight
    query heads per KV head, one rank of eight of a 32 x 131,072 batch: 32 parts 111 us, 37 parts 106 us.)
    """
    tiles = rows * heads_kv
    if tiles < 1 or sms < 1:
        return 1
    return max(1, min(max_splits, (ctas_per_sm * sms) // tiles))


@functools.lru_cache(maxsize=None)
def _multiprocessor_count(device_index: int) -> int:
    return torch.cuda.get_device_properties(device_index).multi_processor_count


def _require_cuda_tensor(tensor: torch.Tensor, name: str, *, device) -> None:
    if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda or tensor.device != device:
        raise ValueError(f"{name} must be a CUDA tensor on {device}")


def _check_device_values(bad: torch.Tensor, message: str) -> None:
    if bool(bad.any()):
        raise ValueError(message)


def _p_scale_arguments(scale_format: str = "nvfp4") -> tuple[int, float]:
    """The probability-scale rule and threshold of an NVFP4 launch. MXFP4 has one rule of its own, so
    the NVFP4 overrides in the environment do not apply to it
    (src/nvfp4_decode_kernel/_decode.py:172-180 of OpenBitSys/BitDecoding-FP4)."""
    if scale_format == "mxfp4":
        import os

        if "NVFP4_P_SCALE_MODE" in os.environ or "NVFP4_P_SCALE_DIVISOR" in os.environ:
            raise ValueError("the NVFP4 P-scale overrides do not apply to MXFP4")
        return bdfp4.P_MODE_IDS["amax6"], resolve_p_scale_tau()
    mode, _, _ = resolve_p_scale_environment()
    if mode not in BUILT_P_SCALE_MODES:
        raise NotImplementedError(
            f"probability scale mode {mode!r} is not built; available: {list(BUILT_P_SCALE_MODES)}"
        )
    return bdfp4.P_MODE_IDS[mode], resolve_p_scale_tau()


def _validate(
    *, query_fp4, query_scales, query_fp4_second, query_scales_second, query_padded_bf16,
    key_pages_fp4, key_scales, value_pages_fp4, value_scales, fp4_page_table, seqused_fp4,
    residual_key_pages_bf16, residual_value_pages_bf16, residual_page_ids, seqused_residual,
    seqused_sink, has_bf16, softmax_scale, out, out_indices, trusted_metadata, scale_format, row_order=None,
):
    """Every host-side contract check of the decode entry; returns the derived geometry."""
    if scale_format not in SCALE_FORMATS:
        raise ValueError(f"scale_format must be one of {list(SCALE_FORMATS)}, got {scale_format!r}")
    # scale atoms (512 bytes: 128 rows x 4 groups) along the 128-value contraction axis
    atoms = HEAD_DIM // (4 * SCALE_FORMATS[scale_format])
    if not torch.cuda.is_available():
        raise RuntimeError("decode_fp4 requires CUDA")
    if not math.isfinite(softmax_scale) or softmax_scale <= 0.0:
        raise ValueError("softmax_scale must be finite and positive")
    if query_fp4.ndim != 4:
        raise ValueError("query_fp4 must have shape [rows, 1, heads_q, 64]")
    device = query_fp4.device
    _require_cuda_tensor(query_fp4, "query_fp4", device=device)
    if torch.cuda.get_device_capability(device)[0] != SM100_MAJOR:
        raise RuntimeError("decode_fp4 requires an SM100-family CUDA device")
    fp4_dtype = torch.float4_e2m1fn_x2
    if query_fp4.dtype is not fp4_dtype or not query_fp4.is_contiguous():
        raise ValueError("query_fp4 must be contiguous packed E2M1 FP4")
    if (query_fp4_second is None) != (query_scales_second is None):
        raise ValueError("query_fp4_second and query_scales_second must be provided together")
    if query_fp4_second is not None:
        _require_cuda_tensor(query_fp4_second, "query_fp4_second", device=device)
        if (
            query_fp4_second.dtype is not fp4_dtype
            or not query_fp4_second.is_contiguous()
            or tuple(query_fp4_second.shape) != tuple(query_fp4.shape)
        ):
            raise ValueError("query_fp4_second must match query_fp4 as contiguous packed E2M1 FP4")
    rows, query_length, heads_q, packed = query_fp4.shape
    if rows < 1 or query_length != 1 or packed * 2 != HEAD_DIM:
        raise ValueError("query_fp4 must have shape [rows, 1, heads_q, 64]")
    for tensor, name in (
        (key_pages_fp4, "key_pages_fp4"), (value_pages_fp4, "value_pages_fp4"),
        (query_scales, "query_scales"), (key_scales, "key_scales"), (value_scales, "value_scales"),
        (fp4_page_table, "fp4_page_table"), (seqused_fp4, "seqused_fp4"),
    ):
        _require_cuda_tensor(tensor, name, device=device)
    packed_types = (torch.uint8, fp4_dtype)
    if (
        key_pages_fp4.dtype not in packed_types
        or key_pages_fp4.ndim != 4
        or key_pages_fp4.shape[1] not in CACHE_PAGE_SIZES
        or key_pages_fp4.shape[3] * 2 != HEAD_DIM
    ):
        raise ValueError("key_pages_fp4 must be packed FP4 with shape [pages, 128, heads_kv, 64]")
    page_count, cache_page, heads_kv, _ = key_pages_fp4.shape
    if scale_format == "mxfp4" and cache_page != PAGE_SIZE:
        raise NotImplementedError("MXFP4 is built for 128-token pages only")
    if value_pages_fp4.dtype not in packed_types or tuple(value_pages_fp4.shape) != (
        page_count, heads_kv, HEAD_DIM, cache_page // 2,
    ):
        raise ValueError(f"value_pages_fp4 must be packed FP4 with shape [pages, heads_kv, 128, {cache_page // 2}]")
    for tensor, name, inner in (
        # 128-token pages are token-major; a 64-token page is head-major in memory ([H][64][64])
        (key_pages_fp4, "key_pages_fp4", (heads_kv * 64, 64, 1) if cache_page == PAGE_SIZE else (64, 64 * 64, 1)),
        (value_pages_fp4, "value_pages_fp4", (HEAD_DIM * cache_page // 2, cache_page // 2, 1)),
    ):
        if tensor.stride()[1:] != inner or tensor.stride(0) % 16 or tensor.data_ptr() % 16:
            raise ValueError(f"{name} must be dense within a page with a 16-byte page pitch")
    if heads_kv < 1 or heads_q % heads_kv:
        raise ValueError("heads_q must be divisible by heads_kv")
    ratio = heads_q // heads_kv
    if ratio > PAGE_SIZE:
        raise ValueError("the query-heads-per-KV-head ratio must be at most 128")
    if ratio > MAX_QUERY_HEADS_PER_KV_HEAD:
        raise NotImplementedError(
            f"this build serves at most {MAX_QUERY_HEADS_PER_KV_HEAD} query heads per KV head, got {ratio}"
        )
    expected_query_sf = (32, 4, 1, 4, atoms, heads_kv, rows)
    # scale regions as (pages, 32, 4, 1, 4, atoms, heads) views of [heads][atoms][32][4][4] bytes; a
    # 64-token K page holds two half atoms, (pages, 32, 2, 1, 4, 2, heads) over [heads][2][32][2][4]
    if cache_page == PAGE_SIZE:
        expected_key_sf = expected_value_sf = (page_count, 32, 4, 1, 4, atoms, heads_kv)
        key_sf_strides = value_sf_strides = (16, 4, atoms * 512, 1, 512, atoms * 512)
    else:
        expected_key_sf, key_sf_strides = (page_count, 32, 2, 1, 4, 2, heads_kv), (8, 4, 512, 1, 256, 512)
        expected_value_sf, value_sf_strides = (page_count, 32, 4, 1, 4, 1, heads_kv), (16, 4, 512, 1, 512, 512)
    query_sf_strides = (16, 4, heads_q * atoms * 512, 1, 512, atoms * 512, heads_q * atoms * 512)
    for scales, name in ((query_scales, "query_scales"), (query_scales_second, "query_scales_second")):
        if scales is None:
            continue
        _require_cuda_tensor(scales, name, device=device)
        if tuple(scales.shape) != expected_query_sf:
            raise ValueError(f"{name} must have shape {expected_query_sf}")
        if scales.stride() != query_sf_strides:
            raise ValueError(f"{name} must use the layout returned by quantize_query")
        if scales.storage_offset() != 0 and scales.data_ptr() % 16:
            raise ValueError(f"{name} must start on a 16-byte boundary")
    for scales, name, expected_page_sf, sf_strides in (
        (key_scales, "key_scales", expected_key_sf, key_sf_strides),
        (value_scales, "value_scales", expected_value_sf, value_sf_strides),
    ):
        if tuple(scales.shape) != expected_page_sf:
            raise ValueError(f"{name} must have shape {expected_page_sf}")
        if scales.dtype not in (torch.uint8, torch.float8_e4m3fn if scale_format == "nvfp4" else torch.float8_e8m0fnu):
            raise ValueError(f"{name} must hold the scale bytes of the {scale_format} format")
        if scales.stride()[1:] != sf_strides or scales.stride(0) % 512:
            raise ValueError(f"{name} must use the quantizer's scale layout with a 512-byte aligned page pitch")
    if (
        fp4_page_table.dtype is not torch.int32
        or fp4_page_table.ndim != 2
        or fp4_page_table.shape[0] != rows
        or fp4_page_table.stride(-1) != 1
    ):
        raise ValueError("fp4_page_table must be row-major INT32 with shape [rows, max_pages]")
    if seqused_fp4.dtype is not torch.int32 or tuple(seqused_fp4.shape) != (rows,) or not seqused_fp4.is_contiguous():
        raise ValueError("seqused_fp4 must be contiguous INT32 with shape [rows]")
    entries_per_step = PAGE_SIZE // cache_page
    max_fp4_tokens = fp4_page_table.shape[1] // entries_per_step * PAGE_SIZE
    if not trusted_metadata:
        _check_device_values(
            (seqused_fp4 < 0) | (seqused_fp4 > max_fp4_tokens) | (seqused_fp4 % PAGE_SIZE != 0),
            f"seqused_fp4 values must be page-aligned and in [0, {max_fp4_tokens}]",
        )
        pages_used = (seqused_fp4 // cache_page)[:, None]
        columns = torch.arange(fp4_page_table.shape[1], device=device)[None, :]
        consumed = columns < pages_used
        _check_device_values(
            consumed & ((fp4_page_table < 0) | (fp4_page_table >= page_count)),
            f"fp4_page_table entries a row consumes must lie in [0, {page_count})",
        )

    residual_values = (residual_key_pages_bf16, residual_value_pages_bf16, residual_page_ids, seqused_residual)
    has_residual = any(value is not None for value in residual_values)
    if has_residual and not all(value is not None for value in residual_values):
        raise ValueError(
            "residual_key_pages_bf16, residual_value_pages_bf16, "
            "residual_page_ids, and seqused_residual must be provided together"
        )
    if not has_residual and (seqused_sink is not None or has_bf16 is not None):
        raise ValueError("seqused_sink and has_bf16 need the BF16 residual arguments")
    if has_residual:
        if query_padded_bf16 is None:
            raise ValueError(
                "pre-quantized query with a BF16 residual requires "
                "query_padded_bf16 support; use the BF16 query path"
            )
        _require_cuda_tensor(query_padded_bf16, "query_padded_bf16", device=device)
        expected_padded = (rows, PAGE_SIZE, heads_q, HEAD_DIM)
        if (
            query_padded_bf16.dtype is not torch.bfloat16
            or tuple(query_padded_bf16.shape) != expected_padded
            or not query_padded_bf16.is_contiguous()
        ):
            raise ValueError(f"query_padded_bf16 must be contiguous BF16 with shape {expected_padded}")
        for tensor, name in (
            (residual_key_pages_bf16, "residual_key_pages_bf16"),
            (residual_value_pages_bf16, "residual_value_pages_bf16"),
            (residual_page_ids, "residual_page_ids"),
            (seqused_residual, "seqused_residual"),
        ):
            _require_cuda_tensor(tensor, name, device=device)
        residual_rows = PAGE_SIZE + (SINK_TOKENS if seqused_sink is not None else 0)
        if residual_key_pages_bf16.ndim != 4:
            raise ValueError(
                f"residual_key_pages_bf16 must be contiguous BF16 with shape [pages, {residual_rows}, heads_kv, 128]"
            )
        expected_residual = (residual_key_pages_bf16.shape[0], residual_rows, heads_kv, HEAD_DIM)
        if (
            residual_key_pages_bf16.dtype is not torch.bfloat16
            or tuple(residual_key_pages_bf16.shape) != expected_residual
            or not residual_key_pages_bf16.is_contiguous()
        ):
            raise ValueError(
                f"residual_key_pages_bf16 must be contiguous BF16 with shape [pages, {residual_rows}, heads_kv, 128]"
            )
        if (
            residual_value_pages_bf16.dtype is not torch.bfloat16
            or tuple(residual_value_pages_bf16.shape) != expected_residual
            or not residual_value_pages_bf16.is_contiguous()
        ):
            raise ValueError("residual_value_pages_bf16 must match the residual K cache")
        for tensor, name in (
            (residual_page_ids, "residual_page_ids"), (seqused_residual, "seqused_residual"),
            (seqused_sink, "seqused_sink"),
        ):
            if tensor is None:
                continue
            _require_cuda_tensor(tensor, name, device=device)
            if tensor.dtype is not torch.int32 or tuple(tensor.shape) != (rows,) or not tensor.is_contiguous():
                raise ValueError(f"{name} must be contiguous INT32 with shape [rows]")
        if has_bf16 is not None:
            _require_cuda_tensor(has_bf16, "has_bf16", device=device)
            if has_bf16.dtype is not torch.bool or tuple(has_bf16.shape) != (rows,):
                raise ValueError("has_bf16 must be BOOL with shape [rows]")
        if not trusted_metadata:
            _check_device_values(
                (seqused_residual < 0) | (seqused_residual > PAGE_SIZE),
                f"seqused_residual values must lie in [0, {PAGE_SIZE}]",
            )
            _check_device_values(
                (residual_page_ids < 0) | (residual_page_ids >= expected_residual[0]),
                "residual_page_ids contains an out-of-range physical page ID",
            )
            if seqused_sink is not None:
                _check_device_values(
                    (seqused_sink < 0) | (seqused_sink > SINK_TOKENS),
                    f"seqused_sink values must lie in [0, {SINK_TOKENS}]",
                )
            if has_bf16 is not None:
                _check_device_values(
                    has_bf16 != (seqused_residual > 0), "has_bf16 must agree with seqused_residual > 0"
                )
    if out is not None:
        _require_cuda_tensor(out, "out", device=device)
        if (
            out.dtype is not torch.bfloat16
            or out.ndim != 3
            or tuple(out.shape[1:]) != (heads_q, HEAD_DIM)
            or out.stride()[1:] != (HEAD_DIM, 1)
            or out.shape[0] < rows
        ):
            raise ValueError("out must be BF16 [>= rows, heads_q, 128], dense within a row")
    if out_indices is not None:
        raise NotImplementedError("out_indices (scattered output rows) is not built")
    if row_order is not None:
        _require_cuda_tensor(row_order, "row_order", device=device)
        if row_order.dtype is not torch.int32 or tuple(row_order.shape) != (rows,) or not row_order.is_contiguous():
            raise ValueError("row_order must be contiguous INT32 with shape [rows]")
        if not trusted_metadata:
            _check_device_values(torch.sort(row_order).values != torch.arange(rows, device=device),
                                 "row_order must be a permutation of the rows")
    return device, rows, heads_q, heads_kv, page_count, has_residual


def _fill_args(
    a: "bdfp4.DecodeArgs", *, rows, heads_q, heads_kv, page_count, query_fp4, query_scales, query_fp4_second,
    query_scales_second, query_padded_bf16, key_pages_fp4, key_scales, value_pages_fp4, value_scales,
    fp4_page_table, seqused_fp4, residual_key_pages_bf16, residual_value_pages_bf16, residual_page_ids,
    seqused_residual, seqused_sink, softmax_scale, row_order=None, scale_format: str = "nvfp4",
    tensor_scales=(1.0, 1.0, 1.0), row_splits=None,
) -> None:
    a.rows, a.heads_q, a.heads_kv = rows, heads_q, heads_kv
    a.query_codes, a.query_scales = query_fp4.data_ptr(), query_scales.data_ptr()
    a.query_codes_second, a.query_scales_second = bdfp4.ptr(query_fp4_second), bdfp4.ptr(query_scales_second)
    a.query_padded = bdfp4.ptr(query_padded_bf16)
    a.key_codes, a.key_scales = key_pages_fp4.data_ptr(), key_scales.data_ptr()
    a.value_codes, a.value_scales = value_pages_fp4.data_ptr(), value_scales.data_ptr()
    a.key_codes_pitch, a.key_scales_pitch = key_pages_fp4.stride(0), key_scales.stride(0)
    a.value_codes_pitch, a.value_scales_pitch = value_pages_fp4.stride(0), value_scales.stride(0)
    a.pages = page_count
    a.page_tokens = key_pages_fp4.shape[1]
    a.page_table = fp4_page_table.data_ptr()
    a.page_table_stride = fp4_page_table.stride(0)
    a.max_pages_per_row = fp4_page_table.shape[1]
    a.seqused_fp4 = seqused_fp4.data_ptr()
    if residual_key_pages_bf16 is not None:
        a.tail_key, a.tail_value = residual_key_pages_bf16.data_ptr(), residual_value_pages_bf16.data_ptr()
        a.tail_slot_stride = residual_key_pages_bf16.stride(0)
        a.tail_slots = residual_key_pages_bf16.shape[0]
        a.tail_slot_ids = residual_page_ids.data_ptr()
        a.seqused_residual = seqused_residual.data_ptr()
        a.seqused_sink = bdfp4.ptr(seqused_sink)
    a.softmax_scale = float(softmax_scale)
    a.p_scale_mode, a.p_scale_tau = _p_scale_arguments(scale_format)
    a.row_order = bdfp4.ptr(row_order)
    a.row_splits = bdfp4.ptr(row_splits)
    a.scale_format = bdfp4.FORMAT_MXFP4 if scale_format == "mxfp4" else bdfp4.FORMAT_NVFP4
    a.key_tensor_scale, a.query_tensor_scale, a.value_tensor_scale = (float(x) for x in tensor_scales)


def decode_fp4(
    *, query_fp4, query_scales, query_fp4_second=None, query_scales_second=None, query_padded_bf16,
    key_pages_fp4, key_scales, value_pages_fp4, value_scales, fp4_page_table, seqused_fp4,
    residual_key_pages_bf16=None, residual_value_pages_bf16=None, residual_page_ids=None,
    seqused_residual=None, seqused_sink=None, has_bf16=None, softmax_scale: float, out=None,
    out_indices=None, trusted_metadata: bool = False, validate_only: bool = False,
    scale_format: str = "nvfp4", row_order=None, tensor_scales=(1.0, 1.0, 1.0),
):
    """Validate and launch the unsplit decode; returns BF16 ``[rows, heads_q, 128]`` (a view of
    ``out[:rows]`` when given), or None under ``validate_only``."""
    device, rows, heads_q, heads_kv, page_count, _ = _validate(
        query_fp4=query_fp4, query_scales=query_scales, query_fp4_second=query_fp4_second,
        query_scales_second=query_scales_second, query_padded_bf16=query_padded_bf16,
        key_pages_fp4=key_pages_fp4, key_scales=key_scales, value_pages_fp4=value_pages_fp4,
        value_scales=value_scales, fp4_page_table=fp4_page_table, seqused_fp4=seqused_fp4,
        residual_key_pages_bf16=residual_key_pages_bf16, residual_value_pages_bf16=residual_value_pages_bf16,
        residual_page_ids=residual_page_ids, seqused_residual=seqused_residual, seqused_sink=seqused_sink,
        has_bf16=has_bf16, softmax_scale=softmax_scale, out=out, out_indices=out_indices,
        trusted_metadata=trusted_metadata, scale_format=scale_format, row_order=row_order,
    )
    if validate_only:
        return None
    if out is None:
        out = torch.empty(rows, heads_q, HEAD_DIM, dtype=torch.bfloat16, device=device)
    a = bdfp4.DecodeArgs()
    _fill_args(
        a, rows=rows, heads_q=heads_q, heads_kv=heads_kv, page_count=page_count, query_fp4=query_fp4,
        query_scales=query_scales, query_fp4_second=query_fp4_second, query_scales_second=query_scales_second,
        query_padded_bf16=query_padded_bf16, key_pages_fp4=key_pages_fp4, key_scales=key_scales,
        value_pages_fp4=value_pages_fp4, value_scales=value_scales, fp4_page_table=fp4_page_table,
        seqused_fp4=seqused_fp4, residual_key_pages_bf16=residual_key_pages_bf16,
        residual_value_pages_bf16=residual_value_pages_bf16, residual_page_ids=residual_page_ids,
        seqused_residual=seqused_residual, seqused_sink=seqused_sink, softmax_scale=softmax_scale,
        row_order=row_order, scale_format=scale_format, tensor_scales=tensor_scales,
    )
    a.out, a.out_row_stride = out.data_ptr(), out.stride(0)
    a.num_splits = 1
    bdfp4.decode(a, bdfp4.current_stream(device))
    return out[:rows]


def decode_fp4_split(
    *, query_fp4, query_scales, query_fp4_second=None, query_scales_second=None, key_pages_fp4, key_scales,
    value_pages_fp4, value_scales, fp4_page_table, seqused_fp4, softmax_scale: float, num_splits: int,
    query_padded_bf16=None, residual_key_pages_bf16=None, residual_value_pages_bf16=None,
    residual_page_ids=None, seqused_residual=None, seqused_sink=None, has_bf16=None, out=None,
    split_partial_scratch=None, split_lse_scratch=None, scale_format: str = "nvfp4",
    split_merge_counters=None, row_order=None, tensor_scales=(1.0, 1.0, 1.0), row_splits=None,
):
    """Split-KV decode: ``num_splits`` CTAs per (row, KV head) write FP32 partials and LSEs,
    then one combine launch produces the BF16 output, or, given ``split_merge_counters`` (INT32,
    at least ``rows * heads_kv`` zeros), the last CTA of each (row, KV head) merges them itself.
    Arguments are assumed validated by ``decode_fp4(validate_only=True)``. Supplied scratch makes
    the call allocation-free. ``row_splits`` (INT32 ``[rows]``, each in ``1..num_splits``; no reference
    counterpart) cuts row ``r`` into ``row_splits[r]`` parts only: for ragged batches."""
    device = query_fp4.device
    rows, _, heads_q, _ = query_fp4.shape
    page_count, _, heads_kv, _ = key_pages_fp4.shape
    has_residual = residual_key_pages_bf16 is not None
    device_index = device.index if device.index is not None else torch.cuda.current_device()
    parts = split_partial_count(
        rows, heads_kv, num_splits, residual=has_residual, sms=_multiprocessor_count(device_index)
    )
    need_out, need_lse = parts * rows * heads_q * HEAD_DIM, parts * rows * heads_q
    for scratch, name, need in (
        (split_partial_scratch, "split_partial_scratch", need_out),
        (split_lse_scratch, "split_lse_scratch", need_lse),
    ):
        if scratch is None:
            continue
        if (
            scratch.dtype is not torch.float32
            or scratch.device != device
            or scratch.ndim != 1
            or not scratch.is_contiguous()
            or scratch.storage_offset() != 0
            or scratch.numel() < need
        ):
            raise ValueError(
                f"{name} must be a contiguous 1-D FP32 buffer at storage offset zero with at least {need} elements"
            )
    partial = (
        torch.empty(need_out, dtype=torch.float32, device=device) if split_partial_scratch is None
        else split_partial_scratch
    )
    lse = torch.empty(need_lse, dtype=torch.float32, device=device) if split_lse_scratch is None else split_lse_scratch
    if out is None:
        out = torch.empty(rows, heads_q, HEAD_DIM, dtype=torch.bfloat16, device=device)
    a = bdfp4.DecodeArgs()
    _fill_args(
        a, rows=rows, heads_q=heads_q, heads_kv=heads_kv, page_count=page_count, query_fp4=query_fp4,
        query_scales=query_scales, query_fp4_second=query_fp4_second, query_scales_second=query_scales_second,
        query_padded_bf16=query_padded_bf16, key_pages_fp4=key_pages_fp4, key_scales=key_scales,
        value_pages_fp4=value_pages_fp4, value_scales=value_scales, fp4_page_table=fp4_page_table,
        seqused_fp4=seqused_fp4, residual_key_pages_bf16=residual_key_pages_bf16,
        residual_value_pages_bf16=residual_value_pages_bf16, residual_page_ids=residual_page_ids,
        seqused_residual=seqused_residual, seqused_sink=seqused_sink, softmax_scale=softmax_scale,
        row_order=row_order, scale_format=scale_format, tensor_scales=tensor_scales, row_splits=row_splits,
    )
    if row_splits is not None and (row_splits.dtype is not torch.int32 or row_splits.device != device
                                   or tuple(row_splits.shape) != (rows,) or not row_splits.is_contiguous()):
        raise ValueError("row_splits must be contiguous INT32 CUDA with shape [rows]")
    a.num_splits = num_splits
    a.bf16_split = int(parts > num_splits)
    a.bf16_page_cost = BF16_BLOCK_PAGE_COST if has_residual and parts == num_splits else 0
    a.partial_out, a.partial_lse = partial.data_ptr(), lse.data_ptr()
    stream = bdfp4.current_stream(device)
    if split_merge_counters is not None:
        if (
            split_merge_counters.dtype is not torch.int32
            or split_merge_counters.device != device
            or not split_merge_counters.is_contiguous()
            or split_merge_counters.numel() < rows * heads_kv
        ):
            raise ValueError(
                f"split_merge_counters must be a contiguous INT32 buffer of at least {rows * heads_kv} zeros"
            )
        a.out, a.out_row_stride = out.data_ptr(), out.stride(0)
        a.merge_counters = split_merge_counters.data_ptr()
        bdfp4.decode(a, stream)
        return out[:rows]
    bdfp4.decode(a, stream)
    bdfp4.combine(partial, lse, parts, rows, heads_q, out, out.stride(0), stream)
    return out[:rows]
