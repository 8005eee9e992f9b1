"""The vLLM attention backend of the NVFP4 KV cache.

vLLM asks a backend class a fixed set of questions (which cache dtypes, block sizes, GPUs and feature
combinations it serves; what shape a cache tensor has; which classes build its metadata and run its
layers). This module answers them for a cache whose pages are flat byte blocks: everything that is not
about the FP4 cache is FlashAttention's answer unchanged, because prefill and the metadata base are
FlashAttention's. Same class name, entry point and answers as src/nvfp4_vllm/backend.py:44-151 of
OpenBitSys/BitDecoding-FP4.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

from vllm.config import get_current_vllm_config_or_none
from vllm.v1.attention.backends.flash_attn import FlashAttentionBackend as _Flash

from .guards import NVFP4


@dataclass(frozen=True)
class _CacheFormat:
    """What the kernels behind this backend are built for."""

    page_tokens: int = 128        # V scale groups run along tokens, a whole page at a time: no other block size
    head_size: int = 128
    compute_major: int = 10       # sm_100
    values_per_byte: int = 2      # E2M1
    values_per_scale: int = 16    # one E4M3 byte each

    def bytes_per_vector(self, head_size: int) -> int:
        return head_size // self.values_per_byte + head_size // self.values_per_scale

    def page_bytes(self, block_size: int, num_kv_heads: int, head_size: int) -> int:
        """K and V of one layer's page. vLLM's cache budget (``AttentionSpec.real_page_size_bytes``)
        is computed from the same product and must come out equal."""
        return 2 * block_size * num_kv_heads * self.bytes_per_vector(head_size)


FORMAT = _CacheFormat()
PAGE_SIZE, HEAD_SIZE, SM100 = FORMAT.page_tokens, FORMAT.head_size, FORMAT.compute_major


def nvfp4_page_size_bytes(block_size: int, num_kv_heads: int, head_size: int) -> int:
    return FORMAT.page_bytes(block_size, num_kv_heads, head_size)


def _engine_cache_dtype() -> str | None:
    """``kv_cache_dtype`` of the engine being configured; None when there is none."""
    cache = getattr(get_current_vllm_config_or_none(), "cache_config", None)
    return getattr(cache, "cache_dtype", None)


class NVFP4Backend(_Flash):
    """FP4 decode and FP4 cache writes; FlashAttention for metadata and BF16 prefill."""

    supported_kv_cache_dtypes: ClassVar[list[str]] = list(_Flash.supported_kv_cache_dtypes) + [NVFP4]

    # ---- identity: vLLM finds the backend through AttentionBackendEnum[get_name()] -----------------
    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_impl_cls() -> type:
        from . import impl

        return impl.NVFP4Impl

    @staticmethod
    def get_builder_cls() -> type:
        from . import builder

        return builder.NVFP4MetadataBuilder

    # ---- what is served ----------------------------------------------------------------------------
    @staticmethod
    def get_supported_kernel_block_sizes() -> list[int]:
        return [FORMAT.page_tokens]

    @classmethod
    def supports_block_size(cls, block_size: int | None) -> bool:
        # exactly one page, not "a multiple of": a 256-token block would be cut into two kernel blocks
        return block_size in (None, FORMAT.page_tokens)

    @classmethod
    def supports_compute_capability(cls, capability) -> bool:
        return capability.major == FORMAT.compute_major

    @classmethod
    def supports_kv_connector(cls) -> bool:
        return False  # connectors ship (address, size) ranges; a packed FP4 page is not one tensor of tokens

    @classmethod
    def supports_combination(cls, head_size, dtype, kv_cache_dtype, block_size, use_mla, has_sink, use_sparse,
                             use_mm_prefix, device_capability) -> str | None:
        """A reason to refuse, or None. Only the FP4 cache narrows anything: with another cache dtype
        this class is FlashAttention. (The selector caches the answer per head size and cache dtype.)"""
        if kv_cache_dtype != NVFP4 or head_size == FORMAT.head_size:
            return None
        return f"NVFP4 decode is compiled for head_size {FORMAT.head_size}, got {head_size}"

    # ---- the cache tensor --------------------------------------------------------------------------
    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> tuple[int, ...]:
        if cache_dtype_str == NVFP4:  # [blocks, bytes]: where the four regions sit is layout.py's business
            return num_blocks, FORMAT.page_bytes(block_size, num_kv_heads, head_size)
        return _Flash.get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size,
                                         cache_dtype_str=cache_dtype_str)

    @staticmethod
    def get_kv_cache_stride_order(include_num_layers_dimension: bool = False) -> tuple[int, ...]:
        # vLLM does not say which cache dtype it asks about, and FlashAttention's permutation has the
        # wrong rank for a [blocks, bytes] tensor. Raising NotImplementedError is the protocol's way
        # of saying "no preference": the caller then keeps the identity order.
        if _engine_cache_dtype() == NVFP4:
            raise NotImplementedError
        return _Flash.get_kv_cache_stride_order(include_num_layers_dimension)
