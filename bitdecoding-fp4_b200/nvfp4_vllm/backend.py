"""Attention backend that declares the NVFP4 KV-cache page layout to vLLM
(src/nvfp4_vllm/backend.py:44-151 of OpenBitSys/BitDecoding-FP4)."""

from __future__ import annotations

from typing import ClassVar

import torch
from vllm.config import get_current_vllm_config_or_none
from vllm.v1.attention.backends.flash_attn import FlashAttentionBackend

from .guards import NVFP4

PAGE_SIZE = 128
HEAD_SIZE = 128
SM100 = 10


def _cache_dtype() -> str | None:
    config = get_current_vllm_config_or_none()
    if config is None or config.cache_config is None:
        return None
    return config.cache_config.cache_dtype


def nvfp4_page_size_bytes(block_size: int, num_kv_heads: int, head_size: int) -> int:
    """Bytes one K+V page of one layer occupies: two E2M1 values per byte plus one E4M3 scale byte
    per 16 values. vLLM budgets the cache from the same expression."""
    return 2 * block_size * num_kv_heads * (head_size // 2 + head_size // 16)


class NVFP4Backend(FlashAttentionBackend):
    """Paged NVFP4 KV cache: FlashAttention metadata and BF16 prefill, FP4 decode and cache writes."""

    supported_kv_cache_dtypes: ClassVar[list[str]] = [*FlashAttentionBackend.supported_kv_cache_dtypes, NVFP4]

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"  # vLLM resolves the enum via AttentionBackendEnum[get_name()]

    @staticmethod
    def get_impl_cls() -> type:
        from .impl import NVFP4Impl

        return NVFP4Impl

    @staticmethod
    def get_builder_cls() -> type:
        from .builder import NVFP4MetadataBuilder

        return NVFP4MetadataBuilder

    @staticmethod
    def get_supported_kernel_block_sizes() -> list[int]:
        # V is quantized along the token axis a full page at a time
        return [PAGE_SIZE]

    @classmethod
    def supports_block_size(cls, block_size: int | None) -> bool:
        return block_size is None or block_size == PAGE_SIZE

    @classmethod
    def supports_compute_capability(cls, capability) -> bool:
        return capability.major == SM100

    @classmethod
    def supports_kv_connector(cls) -> bool:
        return False  # a connector moves pages by address and size, not by the packed FP4 layout

    @classmethod
    def supports_combination(cls, head_size: int, dtype: torch.dtype, kv_cache_dtype: str | None,
                             block_size: int | None, use_mla: bool, has_sink: bool, use_sparse: bool,
                             use_mm_prefix: bool, device_capability) -> str | None:
        if kv_cache_dtype == NVFP4 and head_size != HEAD_SIZE:
            return f"NVFP4 decode is compiled for head_size {HEAD_SIZE}, got {head_size}"
        return None

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        if cache_dtype_str != NVFP4:
            return FlashAttentionBackend.get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size,
                                                            cache_dtype_str=cache_dtype_str)
        return (num_blocks, nvfp4_page_size_bytes(block_size, num_kv_heads, head_size))

    @staticmethod
    def get_kv_cache_stride_order(include_num_layers_dimension: bool = False) -> tuple[int, ...]:
        # declining makes the caller fall back to the identity order a flat byte page needs
        if _cache_dtype() == NVFP4:
            raise NotImplementedError
        return FlashAttentionBackend.get_kv_cache_stride_order(include_num_layers_dimension)
