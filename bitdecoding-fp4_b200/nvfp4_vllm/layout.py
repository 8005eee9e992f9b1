"""A vLLM KV-cache block seen as an NVFP4 page (src/nvfp4_vllm/layout.py:33-130 of
OpenBitSys/BitDecoding-FP4).

vLLM hands out one flat byte page per block. The four regions — K codes, K scales, V codes,
V scales — sit one after another inside each block, so every region view has the block pitch as
its page stride and a block stays the self-contained byte range the engine believes it is.
An MXFP4 page has the same code regions and uses the first half of each scale region (one E8M0
atom per head instead of two E4M3 atoms), so a block has the same size in either format.
"""

from __future__ import annotations

import functools

import torch

from nvfp4_decode_kernel.scale_mode import DEFAULT_SCALE_MODE, scale_format

PAGE_SIZE = 128


@functools.lru_cache(maxsize=None)
def region_specs(num_kv_heads: int, head_dim: int, device: str = "cpu",
                 scale_mode: str = DEFAULT_SCALE_MODE) -> tuple[tuple, ...]:
    """(shape within a page, strides within a page, dtype, bytes) of the four regions, in block
    order. The layouts are those the quantizer writes and the decode kernel reads
    (``include/bdfp4.h``)."""
    if head_dim != 128:
        raise ValueError(f"the NVFP4 page layout is defined for head_dim 128, got {head_dim}")
    h = num_kv_heads
    if scale_format(scale_mode) == "mxfp4":
        atoms, scale_type = 1, torch.float8_e8m0fnu
    else:
        atoms, scale_type = 2, torch.float8_e4m3fn
    scale_shape, scale_strides = (32, 4, 1, 4, atoms, h), (16, 4, atoms * 512, 1, 512, atoms * 512)
    return (
        ((PAGE_SIZE, h, 64), (h * 64, 64, 1), torch.uint8, PAGE_SIZE * h * 64),
        (scale_shape, scale_strides, scale_type, h * 1024),
        ((h, head_dim, 64), (head_dim * 64, 64, 1), torch.uint8, h * head_dim * 64),
        (scale_shape, scale_strides, scale_type, h * 1024),
    )


def page_bytes(num_kv_heads: int, head_dim: int, device: str = "cpu") -> int:
    """Bytes one block must provide for all four regions (= 2 * 128 * H * 72)."""
    return sum(spec[3] for spec in region_specs(num_kv_heads, head_dim, device))


def carve(kv_cache: torch.Tensor, num_kv_heads: int, head_dim: int,
          scale_mode: str = DEFAULT_SCALE_MODE) -> tuple[torch.Tensor, ...]:
    """One layer's ``[blocks, bytes]`` cache as (K codes, K scales, V codes, V scales) views."""
    if kv_cache.ndim != 2 or kv_cache.element_size() != 1:
        raise ValueError(f"expected a [blocks, bytes] byte cache, got {tuple(kv_cache.shape)} of {kv_cache.dtype}")
    blocks, pitch = kv_cache.shape
    if kv_cache.stride() != (pitch, 1):
        raise ValueError("the block array must be contiguous")
    specs = region_specs(num_kv_heads, head_dim, str(kv_cache.device), scale_mode)
    required = sum(spec[3] for spec in specs)
    if pitch != required:
        raise ValueError(
            f"a block of {pitch} bytes cannot hold {required} bytes of NVFP4 "
            "page; the backend's page size and this layout disagree"
        )
    flat = kv_cache.view(torch.uint8)
    views, offset = [], kv_cache.storage_offset()
    for shape, strides, dtype, region_bytes in specs:
        typed = flat if dtype is torch.uint8 else flat.view(dtype)
        views.append(typed.as_strided((blocks,) + shape, (pitch,) + strides, offset))
        offset += region_bytes
    return tuple(views)
