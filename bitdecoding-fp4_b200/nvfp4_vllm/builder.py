"""FlashAttention's metadata builder extended with this step's slot assignment
(src/nvfp4_vllm/builder.py of OpenBitSys/BitDecoding-FP4)."""

from __future__ import annotations

import os

import torch
from vllm.config import VllmConfig
from vllm.v1.attention.backend import AttentionCGSupport, CommonAttentionMetadata
from vllm.v1.attention.backends.flash_attn import FlashAttentionMetadata, FlashAttentionMetadataBuilder
from vllm.v1.attention.backends.utils import split_decodes_and_prefills
from vllm.v1.kv_cache_interface import AttentionSpec

from .control import PAGE_SIZE, ControlPlane, split_sequence_length
from .guards import NVFP4, check_supported
from .metadata import NVFP4Metadata
from .write import PageWorkTable

DEBUG_ENV = "NVFP4_DEBUG"
MAX_DECODE_SPLITS = 32


def decode_num_splits(rows: int, num_kv_heads: int, sms: int) -> int:
    """Key partitions of a decode batch, from its width, the KV heads and the SM count only — never
    from a sequence length, so that a captured graph replays correctly at any context.

    With one CTA per (row, KV head, partition), ``fit`` partitions fill the GPU once. The answer is the
    largest power of two within ``min(fit, MAX_DECODE_SPLITS)``, raised to ``fit - 1`` (one CTA per
    row and KV head stays free for the BF16 tail and sink) when that lies strictly between this power
    of two and the next, i.e. costs no extra level in the merge."""
    if rows < 1:
        return 1
    fit = sms // (rows * num_kv_heads)
    capped = min(fit, MAX_DECODE_SPLITS)
    power = 1 << (capped.bit_length() - 1) if capped > 0 else 1
    return fit - 1 if power < fit - 1 < 2 * power else power


def decode_split(common_attn_metadata: CommonAttentionMetadata) -> tuple[int, int]:
    """(rows, tokens) of this step's decode prefix, checked against the host-side copy of the batch's
    query offsets (already materialized by the model runner: no synchronization).

    The read path hands the first ``rows`` requests to the decode kernel, so they must be exactly the
    one-token requests: a prefix of ones, then — when a full graph pads the batch to its captured
    width — only empty rows, and behind the prefix only requests of more than one token. Anything
    else means the batch was not reordered, and is refused loudly here rather than decoded wrongly."""
    rows, _, tokens, _ = split_decodes_and_prefills(common_attn_metadata, decode_threshold=1)
    offsets = common_attn_metadata.query_start_loc_cpu[:common_attn_metadata.num_reqs + 1]
    lengths = torch.diff(offsets).tolist()
    prefix, behind = lengths[:rows], lengths[rows:]
    live = sum(1 for n in prefix if n > 0)
    padded_ones = prefix == [1] * live + [0] * (len(prefix) - live)
    if not padded_ones or any(n <= 1 for n in behind):
        raise ValueError(
            "the NVFP4 read path needs one-token requests at the front of the "
            f"batch, but query lengths are {lengths} with a decode "
            f"prefix of {rows}"
        )
    return rows, tokens


class NVFP4MetadataBuilder(FlashAttentionMetadataBuilder):
    """A pass-through under any other cache dtype; under NVFP4 it advances the slot table once per
    step, builds the page work table and asks vLLM to sort one-token requests to the front."""

    @classmethod
    def get_cudagraph_support(cls, vllm_config: VllmConfig, kv_cache_spec: AttentionSpec) -> AttentionCGSupport:
        cache = vllm_config.cache_config
        if cache is None or cache.cache_dtype != NVFP4:
            return super().get_cudagraph_support(vllm_config, kv_cache_spec)
        # a prefill runs varlen attention over a token count that changes every step
        return AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE

    def __init__(self, kv_cache_spec: AttentionSpec, layer_names: list[str], vllm_config: VllmConfig,
                 device: torch.device) -> None:
        super().__init__(kv_cache_spec, layer_names, vllm_config, device)
        cache = vllm_config.cache_config
        self.nvfp4 = cache is not None and cache.cache_dtype == NVFP4
        self.built_for_capture = False
        self.capturing = False
        if not self.nvfp4:
            self.plane = None
            return
        self.debug = os.environ.get(DEBUG_ENV) == "1"
        self._init_reorder_batch_threshold(1)
        check_supported(vllm_config)
        scheduler = vllm_config.scheduler_config
        self.plane = ControlPlane(max_num_seqs=scheduler.max_num_seqs,
                                  max_num_batched_tokens=scheduler.max_num_batched_tokens, device=device)
        self.work_table = PageWorkTable(max_num_seqs=scheduler.max_num_seqs,
                                        max_num_batched_tokens=scheduler.max_num_batched_tokens, device=device)
        self.num_kv_heads = kv_cache_spec.num_kv_heads
        self.sms = torch.cuda.get_device_properties(device).multi_processor_count

    def build_for_cudagraph_capture(self, common_attn_metadata: CommonAttentionMetadata) -> FlashAttentionMetadata:
        """Metadata for a batch being recorded into a graph; remembers that capture happened so the
        first real step afterwards starts from a clean slot table."""
        self.capturing = True
        try:
            return super().build_for_cudagraph_capture(common_attn_metadata)
        finally:
            self.capturing = False
            if self.nvfp4:
                self.built_for_capture = True

    def build(self, common_prefix_len: int, common_attn_metadata: CommonAttentionMetadata,
              fast_build: bool = False) -> FlashAttentionMetadata:
        base = super().build(common_prefix_len, common_attn_metadata, fast_build)
        if not self.nvfp4:
            return base
        if self.built_for_capture and not self.capturing:
            self.built_for_capture = False
            self.plane.reset()
        outputs = self.plane.prepare(
            block_table=common_attn_metadata.block_table_tensor, seq_lens=common_attn_metadata.seq_lens,
            query_start_loc=common_attn_metadata.query_start_loc, num_reqs=common_attn_metadata.num_reqs,
            num_actual_tokens=common_attn_metadata.num_actual_tokens)
        if self.debug:
            self.plane.raise_for_errors()
        source_tokens, destination_pages = self.work_table.build(
            query_start_loc=common_attn_metadata.query_start_loc, seqused_fp4=outputs.seqused_fp4,
            row_to_slot=outputs.row_to_slot, block_table=common_attn_metadata.block_table_tensor,
            num_reqs=common_attn_metadata.num_reqs, max_query_len=common_attn_metadata.max_query_len)
        decode_rows, decode_tokens = decode_split(common_attn_metadata)
        query_start_loc = common_attn_metadata.query_start_loc
        if decode_tokens:
            query_start_loc = query_start_loc[decode_rows:] - decode_tokens
        _, max_fp4, _ = split_sequence_length(common_attn_metadata.max_seq_len)
        splits = decode_num_splits(decode_rows, self.num_kv_heads, self.sms)
        # A decode batch wider than the GPU holds at once (four CTAs per SM) is launched longest
        # row first; a resident one starts every CTA at once and needs no order.
        row_order = None
        if decode_rows * self.num_kv_heads * (splits + 1) > 4 * self.sms:
            row_order = torch.argsort(outputs.seqused_fp4[:decode_rows], descending=True).to(torch.int32)
        return NVFP4Metadata.from_flash(
            base, outputs, source_tokens=source_tokens, destination_pages=destination_pages,
            decode_prefix_rows=decode_rows, decode_prefix_tokens=decode_tokens,
            prefill_query_start_loc=query_start_loc, decode_page_columns=max(1, max_fp4 // PAGE_SIZE),
            decode_num_splits=splits, decode_row_order=row_order)
