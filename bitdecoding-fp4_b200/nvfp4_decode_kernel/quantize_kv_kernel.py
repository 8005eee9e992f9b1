"""K/V page quantization and BF16 tail writes, backed by ``bdfp4_kv_write``.

Same names, arguments and error behaviour as src/nvfp4_decode_kernel/quantize_kv_kernel.py
of OpenBitSys/BitDecoding-FP4 (``KVCacheWriter`` :791-1038, ``quantize_key_pages`` /
``quantize_value_pages`` :1115-1184); the work happens in hand-written CUDA kernels behind
the C ABI instead of a JIT-compiled CuTeDSL launch, so constructing a writer compiles nothing.
"""

from __future__ import annotations

import torch

import bdfp4

from .scale_mode import DEFAULT_SCALE_MODE, mode_id, scale_format, sf_vec_size

PAGE_SIZE = 128
# 64-token cache pages (no reference counterpart) are served too; the page size is read off the
# shape of the destination regions (or of the BF16 pages given to quantize_*_pages).
CACHE_PAGE_SIZES = (128, 64)
HEAD_DIM = 128
SF_VEC_SIZE = 16
GROUPS_PER_ATOM = 4
KEY_SCALE_GEOMETRIES = ("local", "gaussian_global")
_SCALE_DTYPES = (torch.uint8, torch.float8_e4m3fn, torch.float8_e8m0fnu)


def scale_atoms(extent: int, scale_mode: str) -> int:
    """Four-group scale atoms covering ``extent`` values."""
    return extent // (GROUPS_PER_ATOM * sf_vec_size(scale_mode))


def scale_dtype(scale_mode: str) -> torch.dtype:
    return torch.float8_e8m0fnu if scale_format(scale_mode) == "mxfp4" else torch.float8_e4m3fn


def _dense_strides(shape: tuple) -> tuple:
    strides = [1]
    for extent in reversed(shape[1:]):
        strides.append(strides[-1] * extent)
    return tuple(reversed(strides))


def _validate_destination(pages_fp4, scales, *, heads: int, inner_shape: tuple, rest_k: int,
                          half_atoms: bool = False, inner_strides: tuple | None = None) -> None:
    """Only the page pitch of a destination is free; its interior is the decode kernel's layout."""
    if (
        pages_fp4.dtype is not torch.uint8
        or not pages_fp4.is_cuda
        or tuple(pages_fp4.shape[1:]) != inner_shape
        or pages_fp4.stride()[1:] != (inner_strides or _dense_strides(inner_shape))
        or pages_fp4.stride(0) % 16
    ):
        raise ValueError(
            f"packed destination must be uint8 CUDA pages of {inner_shape}, "
            "dense within a page, 16-byte page pitch"
        )
    # a 64-token K page holds half atoms: 32 rows x 2 column groups x 4 scales
    scale_shape = (32, 2, 1, 4, rest_k, heads) if half_atoms else (32, 4, 1, 4, rest_k, heads)
    scale_strides = (
        (8, 4, rest_k * 256, 1, 256, rest_k * 256) if half_atoms else (16, 4, rest_k * 512, 1, 512, rest_k * 512)
    )
    if (
        scales.dtype not in _SCALE_DTYPES
        or scales.device != pages_fp4.device
        or tuple(scales.shape[1:]) != scale_shape
        or scales.stride()[1:] != scale_strides
        or scales.stride(0) % 16
    ):
        raise ValueError("scale destination must use the quantizer's own scale layout")
    if pages_fp4.shape[0] != scales.shape[0]:
        raise ValueError("packed and scale destinations must have equal pages")


class KVCacheWriter:
    """K/V into FP4 pages and the BF16 tail.

    Built once with what does not change between steps (scale modes, tail buffers
    ``[layers, slots, 128 + sink_tokens, heads, 128]``, the key shift ``[layers, heads, 128]``
    already in the rotated basis, or the ``[4, layers]`` int64 base-address table of a per-layer
    writer); a call passes the source K/V, one layer's four regions, the work table and the row
    metadata. The roles present are those given: K pages with K regions, V pages with V regions,
    tail tokens with tail buffers. A per-layer writer quantizes the same work items for every
    layer from a source holding the layers back to back, and writes no tail.
    """

    def __init__(
        self,
        *,
        regions: tuple,
        key_scale_mode: str = DEFAULT_SCALE_MODE,
        value_scale_mode: str = DEFAULT_SCALE_MODE,
        key_scale_geometry: str = "local",
        rotate_key: bool = False,
        key_shift: torch.Tensor | None = None,
        tail_key: torch.Tensor | None = None,
        tail_value: torch.Tensor | None = None,
        sink_tokens: int = 0,
        destination_bases: torch.Tensor | None = None,
        key_tensor_scale: float = 1.0,
        value_tensor_scale: float = 1.0,
        error_word: torch.Tensor | None = None,
    ) -> None:
        key_packed, key_scales, value_packed, value_scales = regions
        any_packed = key_packed if key_packed is not None else value_packed
        if any_packed is None:
            raise ValueError("a writer needs K or V regions")
        heads = any_packed.shape[2 if key_packed is not None else 1]
        self.heads = heads
        self.page_size = key_packed.shape[1] if key_packed is not None else value_packed.shape[3] * 2
        if self.page_size not in CACHE_PAGE_SIZES:
            raise ValueError(f"cache pages hold {PAGE_SIZE} (or 64) tokens, not {self.page_size}")
        self.key_scale_mode = key_scale_mode
        self.value_scale_mode = value_scale_mode
        formats = (scale_format(key_scale_mode), scale_format(value_scale_mode))
        if key_scale_geometry not in KEY_SCALE_GEOMETRIES:
            raise ValueError(
                f"unknown key_scale_geometry {key_scale_geometry!r}, expected one of "
                f"{list(KEY_SCALE_GEOMETRIES)}"
            )
        if "mxfp4" in formats and key_scale_geometry != "local":
            raise ValueError("MXFP4 pages support local scales only")
        if "mxfp4" in formats and self.page_size != PAGE_SIZE:
            raise NotImplementedError("MXFP4 pages are built for 128 tokens only")
        for name, scale in (("key_tensor_scale", key_tensor_scale), ("value_tensor_scale", value_tensor_scale)):
            if not (scale > 0.0 and scale < float("inf")):
                raise ValueError(f"{name} must be finite and positive")
        self.key_tensor_scale, self.value_tensor_scale = float(key_tensor_scale), float(value_tensor_scale)
        if error_word is not None and (error_word.dtype is not torch.int32 or not error_word.is_cuda
                                       or error_word.numel() < 1):
            raise ValueError("error_word must be an INT32 CUDA tensor")
        # optional INT32 [1]: a work item whose destination lies past the regions is skipped and
        # BDFP4_DEV_BAD_PAGE is OR-ed in here (not in the reference's signature)
        self._error_word = error_word
        if key_scale_geometry != "local":
            raise NotImplementedError("key_scale_geometry='gaussian_global' is not built")
        if key_packed is None and (key_shift is not None or rotate_key):
            raise ValueError("the K transform needs K regions")
        if (tail_key is None) != (tail_value is None):
            raise ValueError("tail_key and tail_value come together")
        if tail_key is not None and destination_bases is not None:
            raise ValueError("a per-layer writer writes no tail")
        device = any_packed.device
        layers = None
        if destination_bases is not None:
            if (
                destination_bases.dtype is not torch.int64
                or destination_bases.device != device
                or not destination_bases.is_contiguous()
                or destination_bases.ndim != 2
                or destination_bases.shape[0] != 4
            ):
                raise ValueError(
                    "destination_bases must be a contiguous int64 [4, layers] "
                    "table of K packed, K scale, V packed and V scale addresses"
                )
            layers = destination_bases.shape[1]
        if tail_key is not None:
            row = (PAGE_SIZE + sink_tokens, heads, HEAD_DIM)
            for name, tensor in (("tail_key", tail_key), ("tail_value", tail_value)):
                if (
                    tensor.dtype is not torch.bfloat16
                    or tensor.device != device
                    or not tensor.is_contiguous()
                    or tensor.ndim != 5
                    or tuple(tensor.shape[2:]) != row
                    or tensor.shape != tail_key.shape
                ):
                    raise ValueError(
                        f"{name} must be contiguous BF16 [layers, slots, "
                        f"{PAGE_SIZE + sink_tokens}, {heads}, {HEAD_DIM}] on {device}"
                    )
            layers = tail_key.shape[0]
        if key_shift is not None:
            if (
                key_shift.dtype not in (torch.float32, torch.bfloat16)
                or key_shift.device != device
                or not key_shift.is_contiguous()
                or tuple(key_shift.shape[1:]) != (heads, HEAD_DIM)
            ):
                raise ValueError(
                    f"key_shift must be contiguous torch.float32 or torch.bfloat16 "
                    f"[layers, *{(heads, HEAD_DIM)}] on {device}"
                )
            if layers is not None and key_shift.shape[0] != layers:
                raise ValueError(f"key_shift has {key_shift.shape[0]} layers, not {layers}")
            layers = key_shift.shape[0]
        self._regions_dtypes = (
            None if key_scales is None else key_scales.dtype,
            None if value_scales is None else value_scales.dtype,
        )
        self.bind_regions(*regions)
        self.writes_tail = tail_key is not None
        self.layers = layers if destination_bases is not None else None
        self.rotate_key = bool(rotate_key)
        self.sink_tokens = int(sink_tokens)
        self._tail_key, self._tail_value = tail_key, tail_value
        self._key_shift, self._bases = key_shift, destination_bases
        self._device = device

    def bind_regions(self, key_pages_fp4, key_scales, value_pages_fp4, value_scales) -> tuple:
        """Check one layer's four regions once; returns them call-ready."""
        dtypes = (
            None if key_scales is None else key_scales.dtype,
            None if value_scales is None else value_scales.dtype,
        )
        if dtypes != self._regions_dtypes:
            raise ValueError(
                f"regions carry scale dtypes {dtypes}, this writer was built for {self._regions_dtypes}"
            )
        if key_pages_fp4 is not None:
            _validate_destination(
                key_pages_fp4, key_scales, heads=self.heads,
                inner_shape=(self.page_size, self.heads, HEAD_DIM // 2),
                rest_k=scale_atoms(HEAD_DIM, self.key_scale_mode), half_atoms=self.page_size == 64,
                # a 64-token K page is head-major in memory: [H][64 tok][64 B] seen as (tok, H, 64)
                inner_strides=(64, 64 * 64, 1) if self.page_size == 64 else None,
            )
        if value_pages_fp4 is not None:
            _validate_destination(
                value_pages_fp4, value_scales, heads=self.heads,
                inner_shape=(self.heads, HEAD_DIM, self.page_size // 2),
                rest_k=scale_atoms(self.page_size, self.value_scale_mode),
            )
        return (key_pages_fp4, key_scales, value_pages_fp4, value_scales)

    def __call__(
        self,
        key: torch.Tensor | None,
        value: torch.Tensor | None,
        regions: tuple,
        source_tokens: torch.Tensor,
        destination_pages: torch.Tensor,
        query_start_loc: torch.Tensor | None = None,
        seq_lens: torch.Tensor | None = None,
        seqused_fp4: torch.Tensor | None = None,
        row_to_slot: torch.Tensor | None = None,
        layer: int = 0,
        decode_rows: int = 0,
        first_row: int = 0,
    ) -> None:
        """Write this call's pages and tail tokens; launch nothing if there are none.

        ``key`` / ``value`` are ``[tokens, heads, 128]`` BF16, dense within a token. Rows
        ``[0, decode_rows)`` of the row metadata are one-token rows; rows before ``first_row``
        get no tail write.
        """
        if not destination_pages.shape[0] and (not self.writes_tail or seq_lens.shape[0] == first_row):
            return
        source = key if key is not None else value
        for name, tensor in (("key", key), ("value", value)):
            if tensor is None:
                continue
            if (
                tensor.dtype is not torch.bfloat16
                or not tensor.is_cuda
                or tensor.ndim != 3
                or tuple(tensor.shape[1:]) != (self.heads, HEAD_DIM)
                or tensor.stride()[1:] != (HEAD_DIM, 1)
                or tensor.stride(0) % 8
            ):
                raise ValueError(f"{name} must be BF16 CUDA [tokens, {self.heads}, {HEAD_DIM}], dense within a token")
        if self.layers is not None and source.shape[0] % self.layers:
            raise ValueError(
                f"a source of {source.shape[0]} tokens does not divide into {self.layers} layers"
            )
        for name, tensor in (("source_tokens", source_tokens), ("destination_pages", destination_pages)):
            if tensor.dtype is not torch.int32 or not tensor.is_cuda or not tensor.is_contiguous() or tensor.ndim != 1:
                raise ValueError(f"{name} must be contiguous 1-D INT32 CUDA")
        if source_tokens.shape != destination_pages.shape:
            raise ValueError("source_tokens and destination_pages must have equal length")
        key_packed, key_scales, value_packed, value_scales = regions
        a = bdfp4.KvWriteArgs()
        a.key, a.value = bdfp4.ptr(key), bdfp4.ptr(value)
        a.key_token_pitch = key.stride(0) if key is not None else 0
        a.value_token_pitch = value.stride(0) if value is not None else 0
        a.source_tokens_total = source.shape[0]
        a.heads = self.heads
        a.key_codes, a.key_scales = bdfp4.ptr(key_packed), bdfp4.ptr(key_scales)
        a.value_codes, a.value_scales = bdfp4.ptr(value_packed), bdfp4.ptr(value_scales)
        a.key_codes_pitch = key_packed.stride(0) if key_packed is not None else 0
        a.key_scales_pitch = key_scales.stride(0) if key_scales is not None else 0
        a.value_codes_pitch = value_packed.stride(0) if value_packed is not None else 0
        a.value_scales_pitch = value_scales.stride(0) if value_scales is not None else 0
        a.bases = bdfp4.ptr(self._bases)
        a.layers = self.layers or 1
        a.source_tokens, a.destination_pages = bdfp4.ptr(source_tokens), bdfp4.ptr(destination_pages)
        a.work_items = destination_pages.shape[0]
        a.key_scale_mode, a.value_scale_mode = mode_id(self.key_scale_mode), mode_id(self.value_scale_mode)
        a.rotate_key = int(self.rotate_key)
        a.key_shift = bdfp4.ptr(self._key_shift)
        a.key_shift_type = (
            bdfp4.SHIFT_NONE if self._key_shift is None
            else bdfp4.SHIFT_F32 if self._key_shift.dtype is torch.float32 else bdfp4.SHIFT_BF16
        )
        a.layer = int(layer)
        a.page_tokens = self.page_size
        # a destination at or past the regions' page count is skipped and reported, never written
        a.pages = (key_packed if key_packed is not None else value_packed).shape[0]
        a.key_tensor_scale, a.value_tensor_scale = self.key_tensor_scale, self.value_tensor_scale
        a.error_word = bdfp4.ptr(self._error_word)
        if self.writes_tail:
            if any(t is None for t in (query_start_loc, seq_lens, seqused_fp4, row_to_slot)):
                raise ValueError("a tail-writing call needs query_start_loc, seq_lens, seqused_fp4 and row_to_slot")
            a.tail_key, a.tail_value = bdfp4.ptr(self._tail_key), bdfp4.ptr(self._tail_value)
            a.tail_layer_stride = self._tail_key.stride(0)
            a.tail_slot_stride = self._tail_key.stride(1)
            a.sink_tokens = self.sink_tokens
            a.query_start_loc, a.seq_lens = bdfp4.ptr(query_start_loc), bdfp4.ptr(seq_lens)
            a.seqused_fp4, a.row_to_slot = bdfp4.ptr(seqused_fp4), bdfp4.ptr(row_to_slot)
            a.rows = seq_lens.shape[0]
            a.decode_rows, a.first_row = int(decode_rows), int(first_row)
        bdfp4.kv_write(a, bdfp4.current_stream(self._device))


def _validate_pages(pages: torch.Tensor, name: str) -> tuple[int, int, int]:
    if pages.dtype is not torch.bfloat16 or not pages.is_cuda or not pages.is_contiguous() or pages.ndim != 4:
        raise ValueError(f"{name} must be contiguous BF16 CUDA with shape [pages, 128, heads, 128]")
    page_count, page_size, heads, head_dim = pages.shape
    if page_count < 1 or page_size not in CACHE_PAGE_SIZES or head_dim != HEAD_DIM:
        raise ValueError(f"{name} must have shape [pages, 128, heads, 128]")
    return page_count, heads, page_size


def _allocate_scales(page_count: int, heads: int, rest_m: int, rest_k: int, device):
    """Flat storage plus the strided ``(pages,32,4,rest_m,4,rest_k,heads)`` view the kernels use."""
    atom_bytes = 512
    m_block_stride = rest_k * atom_bytes
    head_stride = rest_m * m_block_stride
    page_stride = heads * head_stride
    storage = torch.empty(page_count * page_stride, dtype=torch.uint8, device=device)
    view = storage.as_strided(
        (page_count, 32, 4, rest_m, 4, rest_k, heads),
        (page_stride, 16, 4, m_block_stride, 1, atom_bytes, head_stride),
    )
    return storage, view


def _identity_work(page_count: int, device, page_size: int = PAGE_SIZE):
    pages = torch.arange(page_count, dtype=torch.int32, device=device)
    return pages * page_size, pages


def quantize_key_pages(key_pages: torch.Tensor, scale_mode: str = DEFAULT_SCALE_MODE,
                       scale_geometry: str = "local"):
    """BF16 K pages ``[pages,128,H,128]`` -> fresh E2M1 ``[pages,128,H,64]`` u8 and their scales
    (``[pages,64,H,128]`` -> ``[pages,64,H,64]`` for 64-token pages)."""
    page_count, heads, page_size = _validate_pages(key_pages, "key_pages")
    rest_k = scale_atoms(HEAD_DIM, scale_mode)
    if page_size == PAGE_SIZE:
        key_pages_fp4 = torch.empty(page_count, page_size, heads, HEAD_DIM // 2, dtype=torch.uint8,
                                    device=key_pages.device)
        _, key_scales = _allocate_scales(page_count, heads, 1, rest_k, key_pages.device)
    else:
        key_pages_fp4 = torch.empty(page_count, heads, page_size, HEAD_DIM // 2, dtype=torch.uint8,
                                    device=key_pages.device).permute(0, 2, 1, 3)
        storage = torch.empty(page_count * heads * rest_k * 256, dtype=torch.uint8, device=key_pages.device)
        key_scales = storage.as_strided(
            (page_count, 32, 2, 1, 4, rest_k, heads),
            (heads * rest_k * 256, 8, 4, rest_k * 256, 1, 256, rest_k * 256),
        )
    regions = (key_pages_fp4, key_scales, None, None)
    writer = KVCacheWriter(regions=regions, key_scale_mode=scale_mode, key_scale_geometry=scale_geometry)
    writer(key_pages.reshape(-1, heads, HEAD_DIM), None, regions,
           *_identity_work(page_count, key_pages.device, page_size))
    return key_pages_fp4, key_scales.view(scale_dtype(scale_mode))


def quantize_value_pages(value_pages: torch.Tensor, scale_mode: str = DEFAULT_SCALE_MODE):
    """BF16 V pages ``[pages,128,H,128]`` -> fresh E2M1 ``[pages,H,128,64]`` u8 and their scales
    (``[pages,64,H,128]`` -> ``[pages,H,128,32]`` for 64-token pages)."""
    page_count, heads, page_size = _validate_pages(value_pages, "value_pages")
    rest_k = scale_atoms(page_size, scale_mode)
    value_pages_fp4 = torch.empty(page_count, heads, HEAD_DIM, page_size // 2, dtype=torch.uint8,
                                  device=value_pages.device)
    _, value_scales = _allocate_scales(page_count, heads, HEAD_DIM // 128, rest_k, value_pages.device)
    regions = (None, None, value_pages_fp4, value_scales)
    writer = KVCacheWriter(regions=regions, value_scale_mode=scale_mode)
    writer(None, value_pages.reshape(-1, heads, HEAD_DIM), regions,
           *_identity_work(page_count, value_pages.device, page_size))
    return value_pages_fp4, value_scales.view(scale_dtype(scale_mode))
