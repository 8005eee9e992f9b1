"""Sealing a filled BF16 tail page into the FP4 cache (src/nvfp4_vllm/promote.py:28-48 of
OpenBitSys/BitDecoding-FP4).

V's scale groups run along a page's 128 tokens, so a partial page cannot be quantized; the step
that brings a tail to exactly one page seals it into the block the engine already reserved. One
launch per step over the whole slot table and every layer (rows that did not fill a page carry -1),
after the last layer's attention: by then every layer has read the tail as this step's metadata
describes it and written its share of the token that filled the page.
"""

from __future__ import annotations


def launch(metadata, runtime) -> None:
    """Quantize every filled tail page into its block, for every layer, in one call."""
    writer, regions = runtime.promotion_writer()
    writer(runtime.tail_key_tokens, runtime.tail_value_tokens, regions, metadata.promotion_source_tokens,
           metadata.promotion_pages)
