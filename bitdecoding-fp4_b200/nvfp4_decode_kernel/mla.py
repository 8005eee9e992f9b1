"""MLA latent-cache decode: one compressed KV shared by every query head.

OpenBitSys/BitDecoding-FP4 has no MLA code (src/nvfp4_vllm/backend.py:102 forwards ``use_mla``
and nothing consumes it; head_dim is pinned to 128 at backend.py:112-117), so the interface here
is this package's own, shaped like the GQA one (``fp4_decode`` / ``KVCacheWriter``).

A token is a 512-channel latent and a 64-channel BF16 rope key. A cache page holds 64 tokens in
one block of :data:`BLOCK_BYTES` bytes:

    offset      0  latent codes, scales along channels  [4 chunks][64 tok][64 B]     16384
    offset  16384  their E4M3 scales                    [4 chunks][2][32][2][4]       2048
    offset  18432  latent codes, scales along tokens    [4 chunks][128 ch][32 B]     16384
    offset  34816  their E4M3 scales                    [4 chunks][32][4][4]          2048
    offset  36864  rope keys, BF16                      [64 tok][128 B], 128 B swizzle  8192

The first four regions are exactly what the GQA page writer produces for four KV heads of
64-token pages with the latent given as both key and value; the score product reads the first
copy and the output product the second (704 bytes per token in all).
"""

from __future__ import annotations

import torch

import bdfp4

from .p_scale import DEFAULT_P_SCALE_MODE, P_SMALL_GROUP_AMAX
from .scale_mode import mode_id

PAGE_TOKENS = 64
LATENT = 512
ROPE = 64
CHUNKS = LATENT // 128
REGION_OFFSETS = (0, 16384, 18432, 34816, 36864)
BLOCK_BYTES = 45056
HEADS_PER_CTA = 64


class MLACache:
    """Views over a flat ``[pages, >= BLOCK_BYTES]`` u8 CUDA tensor (row pitch a multiple of 16)."""

    def __init__(self, blocks: torch.Tensor) -> None:
        if blocks.dtype is not torch.uint8 or not blocks.is_cuda or blocks.ndim != 2:
            raise ValueError("an MLA cache is a 2-D uint8 CUDA tensor of page blocks")
        if blocks.shape[1] < BLOCK_BYTES or blocks.stride(1) != 1 or blocks.stride(0) % 16 or blocks.data_ptr() % 16:
            raise ValueError(f"page blocks hold at least {BLOCK_BYTES} bytes at a 16-byte aligned pitch")
        self.blocks = blocks
        sizes = (16384, 2048, 16384, 2048, 8192)
        self.key_codes, self.key_scales, self.value_codes, self.value_scales, self.rope = (
            blocks[:, offset:offset + size] for offset, size in zip(REGION_OFFSETS, sizes))

    @classmethod
    def allocate(cls, pages: int, device) -> "MLACache":
        return cls(torch.zeros(pages, BLOCK_BYTES, dtype=torch.uint8, device=device))

    @property
    def pages(self) -> int:
        return self.blocks.shape[0]

    @property
    def pitch(self) -> int:
        return self.blocks.stride(0)


def _check_work(source_tokens: torch.Tensor, destination_pages: torch.Tensor) -> None:
    for name, tensor in (("source_tokens", source_tokens), ("destination_pages", destination_pages)):
        if tensor.dtype is not torch.int32 or not tensor.is_cuda or not tensor.is_contiguous() or tensor.ndim != 1:
            raise ValueError(f"{name} must be contiguous 1-D INT32 CUDA")
    if source_tokens.shape != destination_pages.shape:
        raise ValueError("source_tokens and destination_pages must have equal length")


def write_pages(cache: MLACache, latent: torch.Tensor, rope: torch.Tensor, source_tokens: torch.Tensor,
                destination_pages: torch.Tensor, *, key_scale_mode: str = "amax6",
                value_scale_mode: str = "amax6") -> None:
    """Quantize whole pages: work item ``i`` takes tokens ``source_tokens[i] .. +63`` of ``latent``
    ``[tokens, 512]`` and ``rope`` ``[tokens, 64]`` (BF16) into page ``destination_pages[i]``
    (negative: skipped). Both latent copies and the rope block are written."""
    _check_work(source_tokens, destination_pages)
    if latent.dtype is not torch.bfloat16 or not latent.is_cuda or latent.ndim != 2 or latent.shape[1] != LATENT \
            or latent.stride(1) != 1 or latent.stride(0) % 8:
        raise ValueError("latent must be BF16 CUDA [tokens, 512], dense within a token")
    if rope.dtype is not torch.bfloat16 or not rope.is_cuda or rope.shape != (latent.shape[0], ROPE) \
            or rope.stride(1) != 1 or rope.stride(0) % 8:
        raise ValueError("rope must be BF16 CUDA [tokens, 64], dense within a token")
    if not destination_pages.numel():
        return
    stream = bdfp4.current_stream(latent.device)
    a = bdfp4.KvWriteArgs()
    a.key = a.value = latent.data_ptr()
    a.key_token_pitch = a.value_token_pitch = latent.stride(0)
    a.source_tokens_total = latent.shape[0]
    a.heads = CHUNKS
    a.key_codes, a.key_scales = cache.key_codes.data_ptr(), cache.key_scales.data_ptr()
    a.value_codes, a.value_scales = cache.value_codes.data_ptr(), cache.value_scales.data_ptr()
    a.key_codes_pitch = a.key_scales_pitch = a.value_codes_pitch = a.value_scales_pitch = cache.pitch
    a.layers = 1
    a.source_tokens, a.destination_pages = source_tokens.data_ptr(), destination_pages.data_ptr()
    a.work_items = destination_pages.numel()
    a.key_scale_mode, a.value_scale_mode = mode_id(key_scale_mode), mode_id(value_scale_mode)
    a.key_shift_type = bdfp4.SHIFT_NONE
    a.page_tokens = PAGE_TOKENS
    a.pages = cache.pages
    bdfp4.kv_write(a, stream)
    check = bdfp4.check
    check("bdfp4_mla_write_rope",
          bdfp4.library().bdfp4_mla_write_rope(rope.data_ptr(), rope.stride(0), source_tokens.data_ptr(),
                                               destination_pages.data_ptr(), destination_pages.numel(),
                                               cache.rope.data_ptr(), cache.pitch, stream))


class MLAAppender:
    """Quantize-on-write of one token per row and step. The rows' open pages (the last, partly filled
    page of each sequence) are kept in BF16 staging buffers; a step puts every row's new token into
    its open page and re-quantizes that page into the cache, so the cache always holds every token in
    NVFP4 (there is no BF16 window in the MLA path). Three launches, no allocation, no host read."""

    def __init__(self, rows: int, device, *, key_scale_mode: str = "amax6", value_scale_mode: str = "amax6") -> None:
        self.rows = rows
        self.latent = torch.zeros(rows * PAGE_TOKENS, LATENT, dtype=torch.bfloat16, device=device)
        self.rope = torch.zeros(rows * PAGE_TOKENS, ROPE, dtype=torch.bfloat16, device=device)
        self.source_tokens = torch.zeros(rows, dtype=torch.int32, device=device)
        self.destination_pages = torch.full((rows,), -1, dtype=torch.int32, device=device)
        self.key_scale_mode, self.value_scale_mode = key_scale_mode, value_scale_mode

    def load_open_pages(self, latent: torch.Tensor, rope: torch.Tensor) -> None:
        """Seed the staging buffers (``[rows, 64, 512]`` / ``[rows, 64, 64]`` BF16, zero past each row's
        length) when sequences enter with a partly filled last page, e.g. after prefill."""
        self.latent.copy_(latent.reshape(self.rows * PAGE_TOKENS, LATENT))
        self.rope.copy_(rope.reshape(self.rows * PAGE_TOKENS, ROPE))

    def append(self, cache: MLACache, new_latent: torch.Tensor, new_rope: torch.Tensor, seq_lens: torch.Tensor,
               page_table: torch.Tensor, error_word: torch.Tensor | None = None) -> None:
        """``new_latent [rows, 512]``, ``new_rope [rows, 64]`` BF16 become token ``seq_lens[r]`` of row
        ``r`` (``seq_lens`` = the lengths before this step; the caller advances them afterwards)."""
        if new_latent.dtype is not torch.bfloat16 or new_latent.shape != (self.rows, LATENT) or not new_latent.is_contiguous() \
                or new_rope.dtype is not torch.bfloat16 or new_rope.shape != (self.rows, ROPE) or not new_rope.is_contiguous():
            raise ValueError("new_latent is contiguous BF16 [rows, 512], new_rope contiguous BF16 [rows, 64]")
        if seq_lens.dtype is not torch.int32 or seq_lens.shape != (self.rows,) or page_table.dtype is not torch.int32 \
                or page_table.ndim != 2 or page_table.shape[0] != self.rows or page_table.stride(1) != 1:
            raise ValueError("seq_lens is INT32 [rows], page_table INT32 [rows, max_pages]")
        stream = bdfp4.current_stream(new_latent.device)
        bdfp4.check("bdfp4_mla_append", bdfp4.library().bdfp4_mla_append(
            new_latent.data_ptr(), new_rope.data_ptr(), self.latent.data_ptr(), self.rope.data_ptr(),
            seq_lens.data_ptr(), page_table.data_ptr(), page_table.stride(0), page_table.shape[1], self.rows,
            cache.pages,
            self.source_tokens.data_ptr(), self.destination_pages.data_ptr(), bdfp4.ptr(error_word), stream))
        write_pages(cache, self.latent, self.rope, self.source_tokens, self.destination_pages,
                    key_scale_mode=self.key_scale_mode, value_scale_mode=self.value_scale_mode)


class MLAScratch:
    """Buffers a decode call would otherwise allocate: query codes and scales, and the split partials.
    Build once per (rows, heads, num_splits) and pass as ``scratch=``; a serving loop then allocates
    nothing per step (and stays capturable in a CUDA graph)."""

    def __init__(self, rows: int, heads: int, num_splits: int, device) -> None:
        self.shape = (rows, heads, num_splits)
        self.codes = torch.empty(rows, heads, LATENT // 2, dtype=torch.uint8, device=device)
        self.scales = torch.empty(rows, heads, LATENT // 16, dtype=torch.uint8, device=device)
        self.partial_out = self.partial_lse = None
        if num_splits > 1:
            self.partial_out = torch.empty(num_splits, rows, heads, LATENT, dtype=torch.float32, device=device)
            self.partial_lse = torch.empty(num_splits, rows, heads, dtype=torch.float32, device=device)


def quantize_query(q_latent: torch.Tensor, scale_mode: str = "amax6", *, out: tuple | None = None):
    """BF16 ``[rows, heads, 512]`` -> ``(codes u8 [rows, heads, 256], scales u8 [rows, heads, 32])``."""
    if q_latent.dtype is not torch.bfloat16 or not q_latent.is_cuda or q_latent.ndim != 3 \
            or q_latent.shape[2] != LATENT or q_latent.stride()[1:] != (LATENT, 1):
        raise ValueError("q_latent must be BF16 CUDA [rows, heads, 512], dense within a row")
    rows, heads, _ = q_latent.shape
    if out is not None:
        codes, scales = out
    else:
        codes = torch.empty(rows, heads, LATENT // 2, dtype=torch.uint8, device=q_latent.device)
        scales = torch.empty(rows, heads, LATENT // 16, dtype=torch.uint8, device=q_latent.device)
    bdfp4.mla_quantize_query(q_latent, mode_id(scale_mode), codes, scales, bdfp4.current_stream(q_latent.device))
    return codes, scales


def mla_decode(q_latent: torch.Tensor, q_rope: torch.Tensor, cache: MLACache, page_table: torch.Tensor,
               seq_lens: torch.Tensor, *, softmax_scale: float, num_splits: int = 1,
               p_scale_mode: str = DEFAULT_P_SCALE_MODE, p_scale_tau: float = P_SMALL_GROUP_AMAX,
               query_scale_mode: str = "amax6", error_word: torch.Tensor | None = None,
               return_partials: bool = False, out: torch.Tensor | None = None, scratch: MLAScratch | None = None):
    """Decode attention of ``q_latent [rows, heads, 512]`` + ``q_rope [rows, heads, 64]`` (BF16; the
    query with the key up-projection absorbed) over the paged latent cache. ``page_table``
    ``[rows, max_pages]`` INT32 lists each row's 64-token pages oldest first, ``seq_lens`` ``[rows]``
    INT32 its tokens. Returns BF16 ``[rows, heads, 512]`` (the value up-projection is the
    caller's), or with ``return_partials`` the FP32 partials and LSEs of the ``num_splits`` parts.
    ``out`` and ``scratch`` (:class:`MLAScratch`) take the place of the per-call allocations."""
    rows, heads, _ = q_latent.shape
    if heads % HEADS_PER_CTA:
        raise NotImplementedError(f"the MLA kernel serves query heads in groups of {HEADS_PER_CTA}")
    if q_rope.dtype is not torch.bfloat16 or q_rope.shape != (rows, heads, ROPE) or not q_rope.is_contiguous():
        raise ValueError("q_rope must be contiguous BF16 [rows, heads, 64]")
    for name, tensor in (("page_table", page_table), ("seq_lens", seq_lens)):
        if tensor.dtype is not torch.int32 or not tensor.is_cuda:
            raise ValueError(f"{name} must be INT32 CUDA")
    if page_table.ndim != 2 or page_table.shape[0] != rows or page_table.stride(1) != 1 or seq_lens.shape != (rows,):
        raise ValueError("page_table is [rows, max_pages], seq_lens is [rows]")
    if num_splits < 1:
        raise ValueError("num_splits must be at least 1")
    device = q_latent.device
    if scratch is not None and scratch.shape != (rows, heads, num_splits):
        raise ValueError(f"scratch was built for (rows, heads, splits) = {scratch.shape}")
    codes, scales = quantize_query(q_latent, query_scale_mode,
                                   out=None if scratch is None else (scratch.codes, scratch.scales))
    a = bdfp4.MlaDecodeArgs()
    a.rows, a.heads_q = rows, heads
    a.query_codes, a.query_scales, a.query_rope = codes.data_ptr(), scales.data_ptr(), q_rope.data_ptr()
    a.key_codes, a.key_scales = cache.key_codes.data_ptr(), cache.key_scales.data_ptr()
    a.value_codes, a.value_scales = cache.value_codes.data_ptr(), cache.value_scales.data_ptr()
    a.key_codes_pitch = a.key_scales_pitch = a.value_codes_pitch = a.value_scales_pitch = cache.pitch
    a.rope_pages, a.rope_pitch = cache.rope.data_ptr(), cache.pitch
    a.pages = cache.pages
    a.page_table, a.page_table_stride = page_table.data_ptr(), page_table.stride(0)
    a.seq_lens = seq_lens.data_ptr()
    a.softmax_scale = float(softmax_scale)
    a.p_scale_mode = bdfp4.P_MODE_IDS[p_scale_mode]
    a.p_scale_tau = float(p_scale_tau)
    a.num_splits = int(num_splits)
    a.error_word = bdfp4.ptr(error_word)
    stream = bdfp4.current_stream(device)
    if out is None:
        out = torch.empty(rows, heads, LATENT, dtype=torch.bfloat16, device=device)
    elif out.dtype is not torch.bfloat16 or out.shape != (rows, heads, LATENT) or not out.is_contiguous():
        raise ValueError("out must be contiguous BF16 [rows, heads, 512]")
    if num_splits == 1 and not return_partials:
        a.out = out.data_ptr()
        bdfp4.mla_decode(a, stream)
        return out
    if scratch is not None and scratch.partial_out is not None:
        partial_out, partial_lse = scratch.partial_out, scratch.partial_lse
    else:
        partial_out = torch.empty(num_splits, rows, heads, LATENT, dtype=torch.float32, device=device)
        partial_lse = torch.empty(num_splits, rows, heads, dtype=torch.float32, device=device)
    a.partial_out, a.partial_lse = partial_out.data_ptr(), partial_lse.data_ptr()
    bdfp4.mla_decode(a, stream)
    if return_partials:
        return partial_out, partial_lse
    bdfp4.mla_combine(partial_out, partial_lse, num_splits, rows, heads, out, stream)
    return out
