"""Per-step attention metadata for the NVFP4 KV cache (src/nvfp4_vllm/metadata.py:27-149 of
OpenBitSys/BitDecoding-FP4): FlashAttention's own metadata plus what the control plane resolved.
Device tensors here are written by the control kernel and must not be read on the host; the plain
ints come from CPU-side batch descriptions."""

from __future__ import annotations

from dataclasses import dataclass, fields

import torch
from vllm.v1.attention.backends.flash_attn import FlashAttentionMetadata

from .control import ControlOutputs


@dataclass(kw_only=True)
class NVFP4Metadata(FlashAttentionMetadata):
    """FlashAttention metadata plus this step's tail-slot assignment."""

    row_to_slot: torch.Tensor  # [num_reqs] int32: tail slot of each batch row, -1 for padding
    token_to_slot: torch.Tensor  # [num_actual_tokens] int32
    seqused_sink: torch.Tensor  # [max_num_seqs] int32, zero for graph-padding rows
    seqused_fp4: torch.Tensor  # [num_reqs] int32: prefix covered by whole FP4 pages
    seqused_residual: torch.Tensor  # [num_reqs] int32: tokens in the BF16 rolling tail
    promotion_source_tokens: torch.Tensor  # [max_num_seqs] int32: first token of each row's tail
    promotion_pages: torch.Tensor  # [max_num_seqs] int32: block to seal the tail into, or -1
    decode_prefix_rows: int  # rows [0, n) emit exactly one token (host int)
    decode_prefix_tokens: int  # where the prefill tokens begin (host int)
    prefill_query_start_loc: torch.Tensor  # [num_prefills + 1] int32, rebased on the first prefill token
    decode_page_columns: int  # page-table columns the decode kernel walks (from the batch's longest row)
    decode_num_splits: int  # split-KV count, chosen from the decode row count alone
    source_tokens: torch.Tensor  # [work] int32: first token of each full page to quantize
    destination_pages: torch.Tensor  # [work] int32: its block, -1 where the grid slot has no work
    # [decode rows] int32, the decode rows longest first (launch order of a batch too wide to be
    # resident at once), or None; not a field of the reference's metadata
    decode_row_order: torch.Tensor | None = None

    @classmethod
    def from_flash(cls, base: FlashAttentionMetadata, outputs: ControlOutputs, *, source_tokens, destination_pages,
                   decode_prefix_rows: int, decode_prefix_tokens: int, prefill_query_start_loc,
                   decode_page_columns: int, decode_num_splits: int,
                   decode_row_order: torch.Tensor | None = None) -> "NVFP4Metadata":
        """Copy every FlashAttention field (the base object is shared by every layer) and append
        the slot fields."""
        return cls(
            **{f.name: getattr(base, f.name) for f in fields(base)},
            row_to_slot=outputs.row_to_slot, token_to_slot=outputs.token_to_slot,
            seqused_sink=outputs.seqused_sink, seqused_fp4=outputs.seqused_fp4,
            seqused_residual=outputs.seqused_residual,
            promotion_source_tokens=outputs.promotion_source_tokens, promotion_pages=outputs.promotion_pages,
            decode_prefix_rows=decode_prefix_rows, decode_prefix_tokens=decode_prefix_tokens,
            prefill_query_start_loc=prefill_query_start_loc, decode_page_columns=decode_page_columns,
            decode_num_splits=decode_num_splits, source_tokens=source_tokens, destination_pages=destination_pages,
            decode_row_order=decode_row_order,
        )
