"""The attention layer vLLM instantiates for ``kv_cache_dtype="nvfp4"``.

A step's batch arrives with its one-token rows sorted to the front. Those rows are decode rows: they
attend over the FP4 pages, the BF16 rolling tail and the sink through ``fp4_decode``. The rows behind
them came with their whole prompt (chunked prefill is refused up front) and attend over this pass's
own BF16 K/V with the engine's FlashAttention, a library call at the boundary of this package; they
never read the cache. Writing the cache is the other half: ``do_kv_cache_update`` quantizes the
step's full pages and puts everything else into the BF16 tail, and after the last layer of a step
the tails that just filled a page are sealed into FP4 blocks.

All GPU state the layers share (tail buffers, scratch, carved cache views, writers) is one
``LayerRuntime`` per model. It has to exist before vLLM measures free memory for the cache, so the
first layer that runs in the profile pass creates it and hands it to its peers.

Class and method names, and the ``nvfp4 cache attestation`` log line, are the drop-in surface of
src/nvfp4_vllm/impl.py of OpenBitSys/BitDecoding-FP4.
"""

from __future__ import annotations

import hashlib
import os

import torch
from vllm.config import get_current_vllm_config
from vllm.forward_context import get_forward_context
from vllm.logger import init_logger
from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl

from nvfp4_decode_kernel.interface import SINK_TOKENS

from . import guards, promote, write
from .runtime import KEY_SHIFT_ENV, LayerRuntime

logger = init_logger(__name__)


def _file_digest(path: str | None) -> str:
    """SHA-256 of a file, ``"none"`` when there is no path."""
    if not path:
        return "none"
    with open(path, "rb") as stream:
        return hashlib.file_digest(stream, "sha256").hexdigest()


def _step_metadata(layer):
    """The metadata vLLM built for ``layer`` this step; None while it profiles memory."""
    from vllm.model_executor.layers.attention.attention import get_attention_context

    return get_attention_context(layer.layer_name)[0]


def _tensor_parallel_slot() -> tuple[int, int]:
    """(size, rank) of this worker's tensor-parallel group, (1, 0) outside one. Only a sidecar needs
    it (a full-model key mean is sliced by rank), so nothing is queried when none is configured."""
    if not os.environ.get(KEY_SHIFT_ENV) or not torch.distributed.is_initialized():
        return 1, 0
    from vllm.distributed import get_tensor_model_parallel_rank, get_tensor_model_parallel_world_size

    return get_tensor_model_parallel_world_size(), get_tensor_model_parallel_rank()


class NVFP4Impl(FlashAttentionImpl):
    """FP4 decode and cache writes under ``kv_cache_dtype="nvfp4"``; FlashAttention's own behaviour
    under any other cache dtype."""

    def __init__(self, *args, **kwargs) -> None:
        config = get_current_vllm_config()
        guards.check_supported(config)  # before super(): an unsupported engine should be told so, not crash later
        super().__init__(*args, **kwargs)
        self.scale_modes = guards.resolve_scale_mode(config)
        self.key_scale_geometry = guards.resolve_key_scale_geometry(config)
        self.query_terms = guards.resolve_query_terms(config)
        self.rotation = guards.resolve_rotation(config)
        guards.check_mxfp4_options(self.scale_modes, key_scale_geometry=self.key_scale_geometry)
        self.nvfp4 = config.cache_config is not None and config.cache_config.cache_dtype == guards.NVFP4
        self.num_slots = 0
        self.runtime: LayerRuntime | None = None
        self.layer_index = 0
        if self.nvfp4:
            guards.check_layer_supported(self)
            self.num_slots = config.scheduler_config.max_num_seqs
            # prefill attends BF16 K/V and decode quantizes the query itself: a BF16 query either way
            self.supports_quant_query_input = False

    # ---- the model's shared state --------------------------------------------------------------
    def _peers(self) -> list:
        """The model's NVFP4 attention modules in the order the forward context lists them; this
        layer must be among them, or its writes could not be coordinated with theirs."""
        modules = [module for module in get_forward_context().no_compile_layers.values()
                   if isinstance(getattr(module, "impl", None), NVFP4Impl)]
        if all(module.impl is not self for module in modules):
            raise ValueError(
                "an NVFP4 layer is running outside the forward context that lists it, so the write path "
                "cannot be shared with its peers")
        return modules

    def _bind_runtime(self, device: torch.device) -> None:
        """Create the shared state (first NVFP4 layer of the profile pass) and number the layers."""
        peers = self._peers()
        shapes = {(m.impl.num_heads, m.impl.num_kv_heads, m.impl.head_size) for m in peers}
        if len(shapes) != 1:
            raise ValueError(f"NVFP4 needs one attention shape across layers, found {shapes}")
        (num_heads, num_kv_heads, head_dim), = shapes
        tp_size, tp_rank = _tensor_parallel_slot()
        runtime = LayerRuntime(
            num_layers=len(peers), num_slots=self.num_slots, num_heads=num_heads, num_kv_heads=num_kv_heads,
            head_dim=head_dim, device=device, query_terms=self.query_terms, rotation=self.rotation,
            key_scale_mode=self.scale_modes.key, value_scale_mode=self.scale_modes.value,
            key_scale_geometry=self.key_scale_geometry, tensor_parallel_size=tp_size, tensor_parallel_rank=tp_rank)
        for index, module in enumerate(peers):
            module.impl.runtime, module.impl.layer_index = runtime, index
        self._attest(runtime, len(peers))

    def _attest(self, runtime: LayerRuntime, layers: int) -> None:
        """One WARN line per engine saying what the cache actually runs with: a scale mode or a
        sidecar that silently failed to arrive would otherwise look exactly like a default."""
        shift = runtime.active_key_shift
        loaded = "none" if shift is None else f"loaded mean_abs={float(shift.abs().mean()):.6g}"
        logger.warning(
            "nvfp4 cache attestation: attention_backend=CUSTOM kv_cache_dtype=nvfp4 key_shift_enabled=%s "
            "key_shift_sha256=%s q_scale_mode=%s k_scale_mode=%s v_scale_mode=%s k_scale_geometry=%s "
            "query_terms=%d sink_tokens=%d layers=%d key_shift=%s",
            shift is not None, _file_digest(os.environ.get(KEY_SHIFT_ENV)), self.scale_modes.query,
            self.scale_modes.key, self.scale_modes.value, runtime.key_scale_geometry, runtime.query_terms,
            SINK_TOKENS, layers, loaded)

    # ---- vLLM's two hooks ------------------------------------------------------------------------
    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping) -> None:
        if not self.nvfp4:
            return super().do_kv_cache_update(layer, key, value, kv_cache, slot_mapping)
        step, runtime, index = _step_metadata(layer), self.runtime, self.layer_index
        if step is None or runtime is None:
            return None  # memory profiling: there is no cache yet
        if index == 0:
            # rows that start a request get their tail pages wiped in every layer before any layer writes
            write.reset_new_request_tails(tail_key=runtime.tail_key, tail_value=runtime.tail_value,
                                          query_start_loc=step.query_start_loc, seq_lens=step.seq_lens,
                                          row_to_slot=step.row_to_slot)
        runtime.measure_keys(index, key, step.num_actual_tokens)  # a no-op unless a calibration is running
        writer, regions = runtime.writer_for(index, kv_cache)
        # decode rows whose new token the query quantizer writes itself (fused tail write) are skipped here
        skip = step.decode_prefix_rows if runtime.decode_writes_tail else 0
        write.write_kv(writer=writer, regions=regions, key=runtime.key_write(index, key)[0], value=value,
                       source_tokens=step.source_tokens, destination_pages=step.destination_pages,
                       query_start_loc=step.query_start_loc, seq_lens=step.seq_lens, seqused_fp4=step.seqused_fp4,
                       row_to_slot=step.row_to_slot, layer_index=index, decode_rows=step.decode_prefix_rows,
                       first_row=skip)
        return None

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                output_block_scale=None):
        if not self.nvfp4:
            return super().forward(layer, query, key, value, kv_cache, attn_metadata, output, output_scale,
                                   output_block_scale)
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("fused output quantization is not supported by the NVFP4 attention path")
        if self.runtime is None:
            self._bind_runtime(query.device)
        step = attn_metadata
        if step is None:
            return output.zero_()  # memory profiling: nothing to attend to, and the residual stream must stay finite
        runtime = self.runtime
        runtime.expect_layer(self.layer_index)
        decode_rows, prefill_from, total = step.decode_prefix_rows, step.decode_prefix_tokens, step.num_actual_tokens
        if decode_rows:
            runtime.attend_decode_rows(self.layer_index, decode_rows, query=query, key=key, value=value,
                                       kv_cache=kv_cache, step=step, out=output, softmax_scale=self.scale,
                                       query_scale_mode=self.scale_modes.query)
        if prefill_from < total:
            self._prefill(prefill_from, query, key, value, step, output)
        if self.layer_index + 1 == runtime.num_layers:
            promote.launch(step, runtime)  # every layer has now read the tails as this step describes them
        return output

    def _decode(self, rows, query, key, value, kv_cache, attn_metadata, output) -> None:
        """The decode rows of this layer (kept under this name for callers of the reference's class)."""
        self.runtime.attend_decode_rows(self.layer_index, rows, query=query, key=key, value=value, kv_cache=kv_cache,
                                        step=attn_metadata, out=output, softmax_scale=self.scale,
                                        query_scale_mode=self.scale_modes.query)

    def _prefill(self, first_token, query, key, value, step, output) -> None:
        """Rows that arrived with their whole prompt: causal varlen FlashAttention over this pass's own
        K/V, so the key offsets are the query offsets and no block table is involved."""
        from vllm.v1.attention.backends.fa_utils import flash_attn_varlen_func

        span = slice(first_token, step.num_actual_tokens)
        offsets, longest = step.prefill_query_start_loc, step.max_query_len
        flash_attn_varlen_func(
            q=query[span], k=key[span], v=value[span], out=output[span], cu_seqlens_q=offsets, cu_seqlens_k=offsets,
            max_seqlen_q=longest, max_seqlen_k=longest, softmax_scale=self.scale, causal=step.causal,
            fa_version=self.vllm_flash_attn_version)
