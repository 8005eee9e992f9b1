"""ctypes binding of ``libbdfp4.so`` (declared in ``include/bdfp4.h``).

The library is the product: there is no Python or CPU fallback. Importing this module
without a built ``lib/libbdfp4.so`` raises, and so does a call that returns a non-zero status.
Build with ``python bitdecoding-fp4_b200/build.py``.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libbdfp4.so"

OK, E_ARG, E_UNSUPPORTED, E_CUDA, E_DEVICE, E_TOO_LARGE = 0, -1, -2, -3, -4, -5
STATIC_SCRATCH_BYTES = 8 << 20
DEV_WAIT_TIMEOUT, DEV_BAD_PAGE = 1, 2
SCALE_MODE_IDS = {"amax6": 0, "four_six": 1, "four_six_sixhalf": 2,
                  "mxfp4_ocp": 3, "mxfp4_round_up": 4, "mxfp4_search": 5}
FORMAT_NVFP4, FORMAT_MXFP4 = 0, 1
P_MODE_IDS = {"amax6": 0, "amax2_or_amax6": 1, "amax2_or_amax6_c8": 2}
SHIFT_NONE, SHIFT_F32, SHIFT_BF16 = 0, 1, 2

EXPORTS = (
    "bdfp4_version",
    "bdfp4_status_string",
    "bdfp4_last_cuda_error",
    "bdfp4_check_device",
    "bdfp4_kv_write",
    "bdfp4_quantize_query",
    "bdfp4_decode",
    "bdfp4_combine",
    "bdfp4_combine_strided",
    "bdfp4_combine_record",
    "bdfp4_decode_split_static",
    "bdfp4_control_step",
    "bdfp4_work_table",
    "bdfp4_tail_reset",
    "bdfp4_key_channel_sums",
    "bdfp4_probability_statistics",
    "bdfp4_mla_quantize_query",
    "bdfp4_mla_write_rope",
    "bdfp4_mla_append",
    "bdfp4_mla_decode",
    "bdfp4_mla_combine",
    "bdfp4_exchange_bytes",
    "bdfp4_peer_alloc",
    "bdfp4_peer_open",
    "bdfp4_peer_close",
    "bdfp4_peer_free",
    "bdfp4_exchange_merge",
)


class LibraryMissingError(RuntimeError):
    """``libbdfp4.so`` has not been built."""


class KvWriteArgs(Structure):
    _fields_ = [
        ("key", c_void_p), ("value", c_void_p),
        ("key_token_pitch", c_int64), ("value_token_pitch", c_int64),
        ("source_tokens_total", c_int64),
        ("heads", c_int32),
        ("key_codes", c_void_p), ("key_scales", c_void_p),
        ("value_codes", c_void_p), ("value_scales", c_void_p),
        ("key_codes_pitch", c_int64), ("key_scales_pitch", c_int64),
        ("value_codes_pitch", c_int64), ("value_scales_pitch", c_int64),
        ("bases", c_void_p), ("layers", c_int32),
        ("source_tokens", c_void_p), ("destination_pages", c_void_p), ("work_items", c_int32),
        ("key_scale_mode", c_int32), ("value_scale_mode", c_int32),
        ("rotate_key", c_int32), ("key_shift", c_void_p), ("key_shift_type", c_int32), ("layer", c_int32),
        ("tail_key", c_void_p), ("tail_value", c_void_p),
        ("tail_layer_stride", c_int64), ("tail_slot_stride", c_int64),
        ("sink_tokens", c_int32),
        ("query_start_loc", c_void_p), ("seq_lens", c_void_p), ("seqused_fp4", c_void_p),
        ("row_to_slot", c_void_p),
        ("rows", c_int32), ("decode_rows", c_int32), ("first_row", c_int32),
        ("error_word", c_void_p),
        ("page_tokens", c_int32),
        ("pages", c_int32),
        ("key_tensor_scale", c_float), ("value_tensor_scale", c_float),
    ]


class QuantizeQueryArgs(Structure):
    _fields_ = [
        ("query", c_void_p), ("query_row_stride", c_int64), ("query_head_stride", c_int64),
        ("row_indices", c_void_p),
        ("rows", c_int32), ("heads_q", c_int32), ("heads_kv", c_int32),
        ("scale_mode", c_int32), ("rotate", c_int32),
        ("query_codes", c_void_p), ("query_scales", c_void_p),
        ("query_codes_second", c_void_p), ("query_scales_second", c_void_p),
        ("query_padded", c_void_p),
        ("new_key", c_void_p), ("new_value", c_void_p),
        ("new_key_token_pitch", c_int64), ("new_value_token_pitch", c_int64),
        ("tail_key", c_void_p), ("tail_value", c_void_p), ("tail_slot_stride", c_int64),
        ("row_to_slot", c_void_p), ("seq_lens", c_void_p), ("seqused_fp4", c_void_p),
        ("rotate_key", c_int32), ("key_shift", c_void_p), ("sink_tokens", c_int32),
        ("tensor_scale", c_float),
    ]


class DecodeArgs(Structure):
    _fields_ = [
        ("rows", c_int32), ("heads_q", c_int32), ("heads_kv", c_int32),
        ("query_codes", c_void_p), ("query_scales", c_void_p),
        ("query_codes_second", c_void_p), ("query_scales_second", c_void_p),
        ("query_padded", c_void_p),
        ("key_codes", c_void_p), ("key_scales", c_void_p),
        ("value_codes", c_void_p), ("value_scales", c_void_p),
        ("key_codes_pitch", c_int64), ("key_scales_pitch", c_int64),
        ("value_codes_pitch", c_int64), ("value_scales_pitch", c_int64),
        ("pages", c_int32),
        ("page_table", c_void_p), ("page_table_stride", c_int64), ("max_pages_per_row", c_int32),
        ("seqused_fp4", c_void_p),
        ("tail_key", c_void_p), ("tail_value", c_void_p), ("tail_slot_stride", c_int64),
        ("tail_slots", c_int32),
        ("tail_slot_ids", c_void_p), ("seqused_residual", c_void_p), ("seqused_sink", c_void_p),
        ("softmax_scale", c_float), ("p_scale_mode", c_int32), ("p_scale_tau", c_float),
        ("out", c_void_p), ("out_row_stride", c_int64),
        ("num_splits", c_int32), ("bf16_split", c_int32),
        ("partial_out", c_void_p), ("partial_lse", c_void_p),
        ("error_word", c_void_p),
        ("bf16_page_cost", c_int32),
        ("page_tokens", c_int32),
        ("merge_counters", c_void_p),
        ("row_order", c_void_p),
        ("scale_format", c_int32),
        ("key_tensor_scale", c_float), ("query_tensor_scale", c_float), ("value_tensor_scale", c_float),
        ("row_splits", c_void_p),
    ]


class MlaDecodeArgs(Structure):
    _fields_ = [
        ("rows", c_int32), ("heads_q", c_int32),
        ("query_codes", c_void_p), ("query_scales", c_void_p), ("query_rope", c_void_p),
        ("key_codes", c_void_p), ("key_scales", c_void_p),
        ("value_codes", c_void_p), ("value_scales", c_void_p),
        ("key_codes_pitch", c_int64), ("key_scales_pitch", c_int64),
        ("value_codes_pitch", c_int64), ("value_scales_pitch", c_int64),
        ("rope_pages", c_void_p), ("rope_pitch", c_int64),
        ("pages", c_int32),
        ("page_table", c_void_p), ("page_table_stride", c_int64),
        ("seq_lens", c_void_p),
        ("softmax_scale", c_float), ("p_scale_mode", c_int32), ("p_scale_tau", c_float),
        ("out", c_void_p),
        ("num_splits", c_int32),
        ("partial_out", c_void_p), ("partial_lse", c_void_p),
        ("error_word", c_void_p),
    ]


class ControlArgs(Structure):
    _fields_ = [
        ("block_table", c_void_p), ("block_table_stride", c_int64), ("block_table_columns", c_int32),
        ("seq_lens", c_void_p), ("query_start_loc", c_void_p),
        ("slot_keys", c_void_p), ("slot_last_seq", c_void_p), ("slot_last_seen", c_void_p), ("step", c_void_p),
        ("row_to_slot", c_void_p), ("token_to_slot", c_void_p),
        ("seqused_sink", c_void_p), ("seqused_fp4", c_void_p), ("seqused_residual", c_void_p),
        ("promotion_source_tokens", c_void_p), ("promotion_pages", c_void_p), ("error_code", c_void_p),
        ("num_reqs", c_int32), ("num_actual_tokens", c_int32), ("num_slots", c_int32), ("sink_tokens", c_int32),
    ]


class ExchangeArgs(Structure):
    """``struct bdfp4_exchange_args``."""

    _fields_ = [
        ("partial_out", c_void_p), ("partial_lse", c_void_p),
        ("parts", c_int32), ("rows", c_int32), ("heads_q", c_int32), ("world", c_int32), ("rank", c_int32),
        ("step", ctypes.c_uint32),
        ("regions", c_void_p * 8),
        ("out", c_void_p), ("out_row_stride", c_int64),
        ("error_word", c_void_p),
    ]


_lib = None


def library() -> ctypes.CDLL:
    """The loaded shared library; raises :class:`LibraryMissingError` when it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise LibraryMissingError(
            f"{LIB_PATH} is missing: build it with `python bitdecoding-fp4_b200/build.py` "
            "(there is no CPU or Python fallback)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.bdfp4_version.restype = c_int32
    lib.bdfp4_status_string.restype = c_char_p
    lib.bdfp4_status_string.argtypes = [c_int32]
    lib.bdfp4_last_cuda_error.restype = c_char_p
    lib.bdfp4_check_device.restype = c_int32
    lib.bdfp4_kv_write.restype = c_int32
    lib.bdfp4_kv_write.argtypes = [POINTER(KvWriteArgs), c_void_p]
    lib.bdfp4_quantize_query.restype = c_int32
    lib.bdfp4_quantize_query.argtypes = [POINTER(QuantizeQueryArgs), c_void_p]
    lib.bdfp4_decode.restype = c_int32
    lib.bdfp4_decode.argtypes = [POINTER(DecodeArgs), c_void_p]
    lib.bdfp4_combine.restype = c_int32
    lib.bdfp4_combine.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_int64, c_void_p]
    lib.bdfp4_combine_record.restype = c_int32
    lib.bdfp4_combine_record.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]
    lib.bdfp4_combine_strided.restype = c_int32
    lib.bdfp4_combine_strided.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_int32, c_int32, c_int32, c_void_p,
                                          c_int64, c_void_p]
    lib.bdfp4_control_step.restype = c_int32
    lib.bdfp4_control_step.argtypes = [POINTER(ControlArgs), c_void_p]
    lib.bdfp4_work_table.restype = c_int32
    lib.bdfp4_work_table.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int32,
                                     c_int32, c_void_p]
    lib.bdfp4_tail_reset.restype = c_int32
    lib.bdfp4_tail_reset.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int64, c_void_p, c_void_p,
                                     c_void_p, c_int32, c_void_p]
    lib.bdfp4_key_channel_sums.restype = c_int32
    lib.bdfp4_key_channel_sums.argtypes = [c_void_p, c_int64, c_int64, c_int32, c_void_p, c_void_p]
    lib.bdfp4_probability_statistics.restype = c_int32
    lib.bdfp4_probability_statistics.argtypes = [c_void_p, c_int64, c_int32, c_int32, c_int32, c_float, c_int32,
                                                 c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.bdfp4_mla_quantize_query.restype = c_int32
    lib.bdfp4_mla_quantize_query.argtypes = [c_void_p, c_int64, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]
    lib.bdfp4_mla_write_rope.restype = c_int32
    lib.bdfp4_mla_write_rope.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_int32, c_void_p, c_int64, c_void_p]
    lib.bdfp4_mla_append.restype = c_int32
    lib.bdfp4_mla_append.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int32,
                                     c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.bdfp4_mla_decode.restype = c_int32
    lib.bdfp4_mla_decode.argtypes = [POINTER(MlaDecodeArgs), c_void_p]
    lib.bdfp4_mla_combine.restype = c_int32
    lib.bdfp4_exchange_bytes.restype = c_int64
    lib.bdfp4_exchange_bytes.argtypes = [c_int32, c_int32, c_int32]
    lib.bdfp4_peer_alloc.restype = c_int32
    lib.bdfp4_peer_alloc.argtypes = [c_int64, POINTER(c_void_p), c_void_p]
    lib.bdfp4_peer_open.restype = c_int32
    lib.bdfp4_peer_open.argtypes = [c_void_p, POINTER(c_void_p)]
    lib.bdfp4_peer_close.restype = c_int32
    lib.bdfp4_peer_close.argtypes = [c_void_p]
    lib.bdfp4_peer_free.restype = c_int32
    lib.bdfp4_peer_free.argtypes = [c_void_p]
    lib.bdfp4_exchange_merge.restype = c_int32
    lib.bdfp4_exchange_merge.argtypes = [POINTER(ExchangeArgs), c_void_p]
    lib.bdfp4_mla_combine.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p]
    lib.bdfp4_decode_split_static.restype = c_int32
    lib.bdfp4_decode_split_static.argtypes = [POINTER(DecodeArgs), c_void_p]
    _lib = lib
    return lib


class KernelError(RuntimeError):
    """A library call returned a non-zero status."""

    def __init__(self, name: str, status: int):
        lib = library()
        text = lib.bdfp4_status_string(status).decode()
        if status == E_CUDA:
            text += ": " + lib.bdfp4_last_cuda_error().decode()
        super().__init__(f"{name} failed with status {status} ({text})")
        self.status = status


def check(name: str, status: int) -> None:
    if status != OK:
        raise KernelError(name, status)


def ptr(tensor) -> int | None:
    """Device (or host) address of a torch tensor, None for None."""
    return None if tensor is None else tensor.data_ptr()


def current_stream(device) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream


def kv_write(args: KvWriteArgs, stream: int) -> None:
    check("bdfp4_kv_write", library().bdfp4_kv_write(ctypes.byref(args), stream))


def quantize_query(args: QuantizeQueryArgs, stream: int) -> None:
    check("bdfp4_quantize_query", library().bdfp4_quantize_query(ctypes.byref(args), stream))


def decode(args: DecodeArgs, stream: int) -> None:
    check("bdfp4_decode", library().bdfp4_decode(ctypes.byref(args), stream))


def combine(partial_out, partial_lse, parts: int, rows: int, heads_q: int, out, out_row_stride: int,
            stream: int) -> None:
    check(
        "bdfp4_combine",
        library().bdfp4_combine(ptr(partial_out), ptr(partial_lse), parts, rows, heads_q, ptr(out),
                                out_row_stride, stream),
    )


def combine_record(partial_out, partial_lse, parts: int, rows: int, heads_q: int, record_out_ptr: int,
                   record_lse_ptr: int, stream: int) -> None:
    """Split-KV partials folded into one FP32 ``[O | LSE]`` partial (addresses given as integers)."""
    check("bdfp4_combine_record",
          library().bdfp4_combine_record(ptr(partial_out), ptr(partial_lse), parts, rows, heads_q, record_out_ptr,
                                         record_lse_ptr, stream))


def combine_strided(partial_out_ptr: int, out_part_stride: int, partial_lse_ptr: int, lse_part_stride: int,
                    parts: int, rows: int, heads_q: int, out, out_row_stride: int, stream: int) -> None:
    check(
        "bdfp4_combine_strided",
        library().bdfp4_combine_strided(partial_out_ptr, out_part_stride, partial_lse_ptr, lse_part_stride, parts,
                                        rows, heads_q, ptr(out), out_row_stride, stream),
    )


def exchange_bytes(world: int, rows: int, heads_q: int) -> int:
    """Bytes of one rank's exchange region for :func:`exchange_merge`."""
    size = int(library().bdfp4_exchange_bytes(world, rows, heads_q))
    if size <= 0:
        raise ValueError(f"no exchange region for world={world}, rows={rows}, heads_q={heads_q}")
    return size


def peer_alloc(size: int) -> tuple[int, bytes]:
    """A zeroed device allocation other processes of this node can map: (address, 64-byte IPC handle)."""
    local = c_void_p()
    handle = ctypes.create_string_buffer(64)
    check("bdfp4_peer_alloc", library().bdfp4_peer_alloc(size, ctypes.byref(local), handle))
    return int(local.value), handle.raw


def peer_open(handle: bytes) -> int:
    """Map another process's :func:`peer_alloc` allocation into this one; returns its address here."""
    mapped = c_void_p()
    check("bdfp4_peer_open", library().bdfp4_peer_open(ctypes.create_string_buffer(handle, 64), ctypes.byref(mapped)))
    return int(mapped.value)


def peer_close(address: int) -> None:
    check("bdfp4_peer_close", library().bdfp4_peer_close(address))


def peer_free(address: int) -> None:
    check("bdfp4_peer_free", library().bdfp4_peer_free(address))


def exchange_merge(args: ExchangeArgs, stream: int) -> None:
    """Fold, send to every rank, wait for every rank, merge: the KV-shard exchange as one launch."""
    check("bdfp4_exchange_merge", library().bdfp4_exchange_merge(ctypes.byref(args), stream))


def decode_split_static(args: DecodeArgs, stream: int) -> None:
    """Split-KV decode + merge whose partial buffers live in the library's own fixed device array
    (``STATIC_SCRATCH_BYTES``): for callers that may not allocate device memory when they decode.
    Raises :class:`KernelError` with ``E_TOO_LARGE`` when the partials would not fit. Calls share
    the array, so run them on one stream; make the first call on a device outside stream capture."""
    check("bdfp4_decode_split_static", library().bdfp4_decode_split_static(ctypes.byref(args), stream))


def mla_quantize_query(query, scale_mode: int, codes, scales, stream: int) -> None:
    """BF16 ``query [rows, heads, 512]`` -> ``codes [rows, heads, 256]`` u8, ``scales [rows, heads, 32]`` u8."""
    rows, heads, _ = query.shape
    check("bdfp4_mla_quantize_query",
          library().bdfp4_mla_quantize_query(ptr(query), query.stride(0), rows, heads, scale_mode, ptr(codes),
                                             ptr(scales), stream))


def mla_write_rope(rope, source_tokens, destination_pages, rope_pages, stream: int) -> None:
    """BF16 ``rope [tokens, 64]``: 64 tokens per work item into the swizzled 8 KB block of its page."""
    check("bdfp4_mla_write_rope",
          library().bdfp4_mla_write_rope(ptr(rope), rope.stride(0), ptr(source_tokens), ptr(destination_pages),
                                         source_tokens.numel(), ptr(rope_pages), rope_pages.stride(0) * 2, stream))


def mla_decode(args: MlaDecodeArgs, stream: int) -> None:
    check("bdfp4_mla_decode", library().bdfp4_mla_decode(ctypes.byref(args), stream))


def mla_combine(partial_out, partial_lse, parts: int, rows: int, heads_q: int, out, stream: int) -> None:
    check("bdfp4_mla_combine",
          library().bdfp4_mla_combine(ptr(partial_out), ptr(partial_lse), parts, rows, heads_q, ptr(out), stream))


def control_step(args: ControlArgs, stream: int) -> None:
    check("bdfp4_control_step", library().bdfp4_control_step(ctypes.byref(args), stream))


def work_table(query_start_loc, seqused_fp4, row_to_slot, block_table, source_tokens, destination_pages,
               num_reqs: int, columns_per_row: int, stream: int) -> None:
    check(
        "bdfp4_work_table",
        library().bdfp4_work_table(ptr(query_start_loc), ptr(seqused_fp4), ptr(row_to_slot), ptr(block_table),
                                   block_table.stride(0), ptr(source_tokens), ptr(destination_pages), num_reqs,
                                   columns_per_row, stream),
    )


def tail_reset(tail_key, tail_value, query_start_loc, seq_lens, row_to_slot, num_reqs: int, stream: int) -> None:
    layers, _, tokens, heads, head_dim = tail_key.shape
    check(
        "bdfp4_tail_reset",
        library().bdfp4_tail_reset(ptr(tail_key), ptr(tail_value), tail_key.stride(0), tail_key.stride(1), layers,
                                   tokens * heads * head_dim, ptr(query_start_loc), ptr(seq_lens), ptr(row_to_slot),
                                   num_reqs, stream),
    )


def key_channel_sums(key, sums, stream: int) -> None:
    """``sums[h][c] += sum_t key[t][h][c]`` in FP64; ``key`` BF16 ``[tokens, H, 128]``, ``sums`` FP64 ``[H, 128]``."""
    tokens, heads, _ = key.shape
    check("bdfp4_key_channel_sums",
          library().bdfp4_key_channel_sums(ptr(key), key.stride(0), tokens, heads, ptr(sums), stream))


def probability_statistics(scores, *, fp4_tokens: int, softmax_scale: float, sink_tokens: int, multiplier: float,
                           page_max_scratch, group_counts, winner_counts, error_sums, oracle_sums,
                           stream: int) -> None:
    """Adds one query position's probability-scale statistics (FP32 ``scores [heads, tokens]``) to the
    per-E4M3-code accumulators; see ``bdfp4_probability_statistics`` in ``include/bdfp4.h``."""
    heads, tokens = scores.shape
    check("bdfp4_probability_statistics",
          library().bdfp4_probability_statistics(
              ptr(scores), scores.stride(0), heads, tokens, fp4_tokens, softmax_scale, sink_tokens, multiplier,
              ptr(page_max_scratch), ptr(group_counts), ptr(winner_counts), ptr(error_sums), ptr(oracle_sums),
              stream))
