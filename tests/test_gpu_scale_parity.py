"""Parity at the sizes the benchmark quotes, on sampled (row, KV head) tiles.

Every other GPU test decodes a few thousand tokens at most. These build the benchmark's own
workloads (tens of thousands of tokens per row through a shuffled block table, the serving recipe:
two query terms, Hadamard, four_six keys, 4 sink + 128 rolling BF16 tokens), decode them once and
compare a handful of independent (row, KV head) tiles with the CPU oracle walking exactly the
cache bytes the kernel read (``oracle/tile_check.py``). Same tolerance as the small cases:
max |err| <= 1e-2, mean relative error <= 1e-3, in BF16.
"""

import pytest
import torch

from oracle import tile_check

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_REL = 1e-2, 1e-3
SINK_USED = 4


def _decode(w, splits):
    from nvfp4_decode_kernel import fp4_decode

    return fp4_decode(
        w.query, *w.regions, w.page_table, w.seqused_fp4, residual_key_pages_bf16=w.tail_key[0],
        residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids,
        seqused_residual=w.seqused_residual, seqused_sink=w.seqused_sink, trusted_metadata=True,
        num_splits=splits, query_terms=2, scale_mode="amax6", query_rotation="hadamard")


def _build(rows, heads_q, heads_kv, context, page_tokens):
    from bdfp4.workload import build_workload

    w = build_workload(rows=rows, heads_q=heads_q, heads_kv=heads_kv, seq_lens=[context] * rows, sink_tokens=16,
                       seed=1000, key_scale_mode="four_six", value_scale_mode="amax6", rotate=True,
                       page_tokens=page_tokens)
    w.seqused_sink.clamp_(max=SINK_USED)
    w.sink_tokens = SINK_USED
    return w


def _gate(w, out, tiles, splits, label):
    from nvfp4_decode_kernel import _decode as decode_module
    from nvfp4_decode_kernel import split_partial_count

    sms = torch.cuda.get_device_properties(0).multi_processor_count
    parts = split_partial_count(w.rows, w.heads_kv, splits, residual=True, sms=sms)
    result = tile_check.check_tiles(w, out, tiles, terms=2, scale_mode="amax6", rotate=True, num_splits=splits,
                                    bf16_split=parts > splits,
                                    bf16_page_cost=decode_module.BF16_BLOCK_PAGE_COST if parts == splits else 0)
    print(f"{label}: {result}")
    assert result["max_abs"] <= MAX_ABS, (label, result)
    assert result["mean_rel"] <= MEAN_REL, (label, result)


@pytest.mark.parametrize("page_tokens", [64, 128])
def test_headline_workload_tiles(page_tokens):
    """64 rows x 65,536 tokens, 32 query / 8 KV heads: the step the benchmark times (no split)."""
    from nvfp4_decode_kernel._decode import resident_num_splits

    w = _build(64, 32, 8, 65536, page_tokens)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    splits = resident_num_splits(w.rows, w.heads_kv, sms=sms)
    out = _decode(w, splits)
    torch.cuda.synchronize()
    _gate(w, out, [(0, 0), (17, 3), (40, 7), (63, 5)], splits, f"headline, {page_tokens}-token pages")


def test_eight_heads_per_group_long_context_tiles():
    """32 rows x 131,072 tokens, 32 query / 4 KV heads (eight query heads per KV head), with the split
    count the benchmark would choose for that batch width."""
    from nvfp4_decode_kernel._decode import resident_num_splits

    w = _build(32, 32, 4, 131072, 64)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    splits = resident_num_splits(w.rows, w.heads_kv, sms=sms)
    out = _decode(w, splits)
    torch.cuda.synchronize()
    _gate(w, out, [(0, 1), (13, 0), (31, 3)], splits, f"G = 8, 131,072 tokens, {splits} splits")


def test_one_rank_of_an_eight_way_head_partition():
    """What one of eight ranks runs when the headline step is partitioned by KV head: 64 rows of one KV
    head, split along KV so that the launch fills the GPU."""
    from nvfp4_decode_kernel._decode import resident_num_splits

    w = _build(64, 4, 1, 65536, 64)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    splits = resident_num_splits(w.rows, w.heads_kv, sms=sms)
    assert splits > 1
    out = _decode(w, splits)
    torch.cuda.synchronize()
    _gate(w, out, [(5, 0), (62, 0)], splits, f"one KV head per rank, {splits} splits")
