"""Attention over the NVFP4 cache, split by what each row is doing (src/nvfp4_vllm/impl.py of
OpenBitSys/BitDecoding-FP4).

vLLM sorts the one-token rows to the front of the batch. That decode prefix reads the FP4 pages and
the BF16 tail through ``fp4_decode``; the prefill suffix attends this pass's own BF16 K/V with
FlashAttention (a library call at the boundary) and never touches the block table.
"""

from __future__ import annotations

import hashlib
import os

import torch
from vllm.config import get_current_vllm_config
from vllm.forward_context import get_forward_context
from vllm.logger import init_logger
from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl

from nvfp4_decode_kernel import DecodeTailWrite, fp4_decode
from nvfp4_decode_kernel.interface import SINK_TOKENS

from . import promote
from .guards import (NVFP4, check_layer_supported, check_mxfp4_options, check_supported,
                     resolve_key_scale_geometry, resolve_query_terms, resolve_rotation, resolve_scale_mode)
from .runtime import KEY_SHIFT_ENV, LayerRuntime
from .write import reset_new_request_tails, write_kv

logger = init_logger(__name__)


def _sidecar_sha256(env_name: str) -> str:
    path = os.environ.get(env_name)
    if not path:
        return "none"
    digest = hashlib.sha256()
    with open(path, "rb") as stream:
        for chunk in iter(lambda: stream.read(1 << 20), b""):
            digest.update(chunk)
    return digest.hexdigest()


def _attention_metadata(layer):
    """This step's metadata of ``layer`` (None during the profile run)."""
    from vllm.model_executor.layers.attention.attention import get_attention_context

    metadata, _, _, _ = get_attention_context(layer.layer_name)
    return metadata


class NVFP4Impl(FlashAttentionImpl):
    """FP4 decode + cache writes for ``kv_cache_dtype="nvfp4"``; plain FlashAttention otherwise."""

    def __init__(self, *args, **kwargs) -> None:
        config = get_current_vllm_config()
        check_supported(config)  # ahead of super(), so an unsupported engine is reported as such
        super().__init__(*args, **kwargs)
        cache = config.cache_config
        self.nvfp4 = cache is not None and cache.cache_dtype == NVFP4
        self.num_slots = 0
        self.scale_modes = resolve_scale_mode(config)
        self.key_scale_geometry = resolve_key_scale_geometry(config)
        self.query_terms = resolve_query_terms(config)
        self.rotation = resolve_rotation(config)
        check_mxfp4_options(self.scale_modes, key_scale_geometry=self.key_scale_geometry)
        if self.nvfp4:
            check_layer_supported(self)
            # both paths need a BF16 query: prefill attends BF16 K/V, decode quantizes to FP4 itself
            self.supports_quant_query_input = False
            self.num_slots = config.scheduler_config.max_num_seqs
        self.runtime: LayerRuntime | None = None
        self.layer_index = 0

    def _bind_runtime(self, device: torch.device) -> None:
        """Create the model's shared state once, during the profile run, and hand it to every
        NVFP4 layer (so the engine subtracts it from the cache budget)."""
        modules = [m for m in get_forward_context().no_compile_layers.values()
                   if isinstance(getattr(m, "impl", None), NVFP4Impl)]
        if not any(m.impl is self for m in modules):
            raise ValueError(
                "an NVFP4 layer is running outside the forward context that "
                "lists it, so the write path cannot be shared with its peers"
            )
        shapes = {(m.impl.num_heads, m.impl.num_kv_heads, m.impl.head_size) for m in modules}
        if len(shapes) != 1:
            raise ValueError(f"NVFP4 needs one attention shape across layers, found {shapes}")
        num_heads, num_kv_heads, head_dim = shapes.pop()
        tp_size, tp_rank = 1, 0
        if os.environ.get(KEY_SHIFT_ENV) and torch.distributed.is_initialized():
            from vllm.distributed import get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size

            tp_size, tp_rank = get_tensor_model_parallel_world_size(), get_tensor_model_parallel_rank()
        runtime = LayerRuntime(
            num_layers=len(modules), num_slots=self.num_slots, num_heads=num_heads, num_kv_heads=num_kv_heads,
            head_dim=head_dim, device=device, query_terms=self.query_terms, rotation=self.rotation,
            key_scale_mode=self.scale_modes.key, value_scale_mode=self.scale_modes.value,
            key_scale_geometry=self.key_scale_geometry, tensor_parallel_size=tp_size, tensor_parallel_rank=tp_rank)
        shift = runtime.active_key_shift
        # a correctness attestation, once per engine, kept visible at WARN: says what the cache is
        # actually running, since a scale mode or sidecar that failed to arrive looks like a default
        logger.warning(
            "nvfp4 cache attestation: attention_backend=CUSTOM kv_cache_dtype=nvfp4 key_shift_enabled=%s "
            "key_shift_sha256=%s q_scale_mode=%s k_scale_mode=%s v_scale_mode=%s k_scale_geometry=%s "
            "query_terms=%d sink_tokens=%d layers=%d key_shift=%s",
            shift is not None, _sidecar_sha256(KEY_SHIFT_ENV), self.scale_modes.query, self.scale_modes.key,
            self.scale_modes.value, runtime.key_scale_geometry, runtime.query_terms, SINK_TOKENS, len(modules),
            "none" if shift is None else f"loaded mean_abs={float(shift.abs().mean()):.6g}")
        for index, module in enumerate(modules):
            module.impl.runtime = runtime
            module.impl.layer_index = index

    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping) -> None:
        if not self.nvfp4:
            super().do_kv_cache_update(layer, key, value, kv_cache, slot_mapping)
            return
        metadata = _attention_metadata(layer)
        if metadata is None or self.runtime is None:
            return  # profile run: no cache to write into
        runtime = self.runtime
        if self.layer_index == 0:
            # a slot's previous tenant is erased from every layer before any of them writes
            reset_new_request_tails(tail_key=runtime.tail_key, tail_value=runtime.tail_value,
                                    query_start_loc=metadata.query_start_loc, seq_lens=metadata.seq_lens,
                                    row_to_slot=metadata.row_to_slot)
        runtime.measure_keys(self.layer_index, key, metadata.num_actual_tokens)  # only while calibrating
        key, _, _ = runtime.key_write(self.layer_index, key)
        writer, regions = runtime.writer_for(self.layer_index, kv_cache)
        decode_rows = metadata.decode_prefix_rows
        write_kv(writer=writer, regions=regions, key=key, value=value, source_tokens=metadata.source_tokens,
                 destination_pages=metadata.destination_pages, query_start_loc=metadata.query_start_loc,
                 seq_lens=metadata.seq_lens, seqused_fp4=metadata.seqused_fp4, row_to_slot=metadata.row_to_slot,
                 layer_index=self.layer_index, decode_rows=decode_rows,
                 first_row=decode_rows if runtime.decode_writes_tail else 0)

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                output_block_scale=None):
        if not self.nvfp4:
            return super().forward(layer, query, key, value, kv_cache, attn_metadata, output, output_scale,
                                   output_block_scale)
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("fused output quantization is not supported by the NVFP4 attention path")
        if self.runtime is None:
            self._bind_runtime(query.device)
        if attn_metadata is None:
            return output.zero_()  # profile run: nothing to read, and NaN must not enter the residual stream
        self.runtime.expect_layer(self.layer_index)
        rows = attn_metadata.decode_prefix_rows
        tokens = attn_metadata.decode_prefix_tokens
        if rows:
            self._decode(rows, query, key, value, kv_cache, attn_metadata, output)
        if tokens < attn_metadata.num_actual_tokens:
            self._prefill(tokens, query, key, value, attn_metadata, output)
        if self.layer_index == self.runtime.num_layers - 1:
            promote.launch(attn_metadata, self.runtime)  # after the last layer read and wrote the tail
        return output

    def _decode(self, rows, query, key, value, kv_cache, attn_metadata, output) -> None:
        """The one-token rows over the FP4 pages and the tail; every per-row argument is a prefix
        slice of this step's arrays."""
        runtime = self.runtime
        key_pages_fp4, key_scales, value_pages_fp4, value_scales = runtime.views(self.layer_index, kv_cache)
        pages = attn_metadata.decode_page_columns
        raw_key, rotate_key, key_shift = runtime.key_write(self.layer_index, key)
        tail_write = None
        if runtime.decode_writes_tail:
            tail_write = DecodeTailWrite(
                key=raw_key[:rows], value=value[:rows], tail_key=runtime.tail_key[self.layer_index],
                tail_value=runtime.tail_value[self.layer_index], row_to_slot=attn_metadata.row_to_slot[:rows],
                seq_lens=attn_metadata.seq_lens[:rows], seqused_fp4=attn_metadata.seqused_fp4[:rows],
                rotate_key=rotate_key, key_shift=key_shift, sink_tokens=SINK_TOKENS)
        fp4_decode(
            query=runtime.transform_query(query[:rows]), key_pages_fp4=key_pages_fp4, key_scales=key_scales,
            value_pages_fp4=value_pages_fp4, value_scales=value_scales,
            fp4_page_table=attn_metadata.block_table[:rows, :pages], seqused_fp4=attn_metadata.seqused_fp4[:rows],
            seqused_sink=attn_metadata.seqused_sink[:rows] if SINK_TOKENS else None,
            residual_key_pages_bf16=runtime.tail_key[self.layer_index],
            residual_value_pages_bf16=runtime.tail_value[self.layer_index],
            residual_page_ids=attn_metadata.row_to_slot[:rows],
            seqused_residual=attn_metadata.seqused_residual[:rows], softmax_scale=self.scale,
            trusted_metadata=True,  # produced on the device this same step; checking would synchronise
            query_padded_scratch=runtime.query_padded, query_fp4_scratch=runtime.query_fp4,
            query_scales_scratch=runtime.query_scales, query_fp4_second_scratch=runtime.query_fp4_second,
            query_scales_second_scratch=runtime.query_scales_second, num_splits=attn_metadata.decode_num_splits,
            split_partial_scratch=runtime.split_partial, split_lse_scratch=runtime.split_lse,
            row_order=attn_metadata.decode_row_order,
            query_terms=runtime.query_terms, scale_mode=self.scale_modes.query,
            query_rotation=runtime.query_rotation, out=output[:rows], tail_write=tail_write)

    def _prefill(self, tokens, query, key, value, attn_metadata, output) -> None:
        """Rows that arrived with their whole prompt: cache-free varlen FlashAttention over this
        pass's own K/V (``cu_seqlens_k`` is ``cu_seqlens_q``)."""
        from vllm.v1.attention.backends.fa_utils import flash_attn_varlen_func

        starts = attn_metadata.prefill_query_start_loc
        end = attn_metadata.num_actual_tokens
        flash_attn_varlen_func(
            q=query[tokens:end], k=key[tokens:end], v=value[tokens:end], out=output[tokens:end],
            cu_seqlens_q=starts, max_seqlen_q=attn_metadata.max_query_len, cu_seqlens_k=starts,
            max_seqlen_k=attn_metadata.max_query_len, softmax_scale=self.scale, causal=attn_metadata.causal,
            fa_version=self.vllm_flash_attn_version)
