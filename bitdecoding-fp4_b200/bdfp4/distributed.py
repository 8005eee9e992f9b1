"""One very long sequence split along the KV axis across GPUs.

The (row, KV head) units of decode attention are independent, so a batch is partitioned over GPUs
by KV-head group and by row with no exchange at all. The one case with an exchange step is a
single sequence too long for one GPU's share of the step time: its FP4 pages are split into
contiguous ranges, one per rank, each rank decodes its range into a normalised FP32 partial and a
natural-log LSE (``bdfp4_decode`` with ``out = NULL``), the ``[O | LSE]`` records are exchanged
with ONE ``all_gather`` (16.5 KB per row at 32 query heads) and every rank merges them with
``bdfp4_combine_strided`` — the LSE-weighted sum of the intra-GPU split path
(src/nvfp4_decode_kernel/split_k_combine.py:62-83 of OpenBitSys/BitDecoding-FP4), which has no
multi-GPU form of its own. Remote records land in local HBM through the collective before the
merge kernel reads them.

The BF16 blocks have exactly one owner each: the rank holding logical page 0 owns the sink (and
masks its duplicate inside page 0), the rank holding the newest pages owns the rolling tail.
"""

from __future__ import annotations

import torch

HEAD_DIM = 128


def shard_pages(total_pages: int, world_size: int, rank: int) -> tuple[int, int]:
    """Pages ``[first, last)`` of ``rank``: contiguous chunks of ``ceil(total / world)``, the rule
    the intra-GPU split uses (src/nvfp4_decode_kernel/_fa4/block_info.py:47-54)."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"invalid shard coordinates: rank={rank}, world_size={world_size}")
    chunk = -(-total_pages // world_size) if total_pages else 0
    first = min(rank * chunk, total_pages)
    return first, min(first + chunk, total_pages)


def record_floats(rows: int, heads_q: int) -> int:
    """Floats in one rank's ``[O | LSE]`` record."""
    return rows * heads_q * (HEAD_DIM + 1)


def split_record(gathered: torch.Tensor, world_size: int, rows: int, heads_q: int):
    """Views of a gathered ``[world * record]`` buffer: partial outputs ``[world, rows, Hq, 128]``
    and LSEs ``[world, rows, Hq]`` (both strided by the record length)."""
    record = record_floats(rows, heads_q)
    table = gathered.view(world_size, record)
    outs = table[:, :rows * heads_q * HEAD_DIM].unflatten(1, (rows, heads_q, HEAD_DIM))
    lses = table[:, rows * heads_q * HEAD_DIM:].unflatten(1, (rows, heads_q))
    return outs, lses


def decode_kv_sharded(query: torch.Tensor, key_pages_fp4, key_scales, value_pages_fp4, value_scales,
                      fp4_page_table: torch.Tensor, seqused_fp4: torch.Tensor, *, group=None,
                      residual_key_pages_bf16=None, residual_value_pages_bf16=None, residual_page_ids=None,
                      seqused_residual=None, seqused_sink=None, softmax_scale: float | None = None,
                      query_terms: int = 2, scale_mode: str = "amax6", query_rotation: str = "none",
                      out: torch.Tensor | None = None, num_splits: int | None = None,
                      workspace: dict | None = None) -> torch.Tensor:
    """Decode attention over a sequence whose FP4 pages are sharded across the ranks of ``group``.

    Every rank passes the same ``query`` and its own shard: local cache regions, a local page table
    and ``seqused_fp4`` counting only its pages. Pass the BF16 residual arguments only on the rank
    that owns them (see the module docstring); with ``seqused_sink`` but ``seqused_residual`` zero a
    rank owns the sink alone. Returns the merged BF16 output on every rank.

    A rank's shard of one long sequence is only ``rows * heads_kv`` independent walks, far fewer than
    the GPU has SMs, so the shard is itself split along KV into ``num_splits`` parts (default: enough
    to keep four CTAs per SM resident, from the batch width alone) whose partials the rank folds into
    its one record before the exchange. ``workspace`` (a dict the caller keeps between steps) holds
    the buffers a call would otherwise allocate; it is tied to the shapes of its first call.
    """
    import torch.distributed as dist

    import bdfp4
    from nvfp4_decode_kernel import _decode
    from nvfp4_decode_kernel._quantize import quantize_query

    world = dist.get_world_size(group)
    rows, heads_q, head_dim = query.shape
    heads_kv = key_pages_fp4.shape[2]
    device = query.device
    has_residual = residual_key_pages_bf16 is not None
    if num_splits is None:
        num_splits = _decode.resident_num_splits(rows, heads_kv, sms=_decode._multiprocessor_count(device.index or 0))
    record = record_floats(rows, heads_q)
    ws = workspace if workspace is not None else {}
    key = (rows, heads_q, world, num_splits, has_residual, device)
    if ws.get("key") != key:
        ws.clear()
        ws["key"] = key
        # rows past the first of each padded query tile stay zero: written once, here
        ws["padded"] = (torch.zeros(rows, 128, heads_q, head_dim, dtype=torch.bfloat16, device=device)
                        if has_residual else None)
        ws["local"] = torch.empty(record, dtype=torch.float32, device=device)
        ws["gathered"] = torch.empty(world * record, dtype=torch.float32, device=device)
        if num_splits > 1:
            ws["partial_out"] = torch.empty(num_splits, rows, heads_q, HEAD_DIM, dtype=torch.float32, device=device)
            ws["partial_lse"] = torch.empty(num_splits, rows, heads_q, dtype=torch.float32, device=device)
    padded = ws["padded"]
    quantized = quantize_query(query, query_padded_out=padded, heads_kv=heads_kv, query_terms=query_terms,
                               scale_mode=scale_mode, rotation=query_rotation)
    second = (quantized[2], quantized[3]) if query_terms == 2 else (None, None)
    args = bdfp4.DecodeArgs()
    _decode._fill_args(
        args, rows=rows, heads_q=heads_q, heads_kv=heads_kv, page_count=key_pages_fp4.shape[0],
        query_fp4=quantized[0], query_scales=quantized[1], query_fp4_second=second[0],
        query_scales_second=second[1], query_padded_bf16=padded, key_pages_fp4=key_pages_fp4,
        key_scales=key_scales, value_pages_fp4=value_pages_fp4, value_scales=value_scales,
        fp4_page_table=fp4_page_table, seqused_fp4=seqused_fp4,
        residual_key_pages_bf16=residual_key_pages_bf16, residual_value_pages_bf16=residual_value_pages_bf16,
        residual_page_ids=residual_page_ids, seqused_residual=seqused_residual, seqused_sink=seqused_sink,
        softmax_scale=softmax_scale if softmax_scale is not None else head_dim ** -0.5)
    local, gathered = ws["local"], ws["gathered"]
    stream = bdfp4.current_stream(device)
    lse_offset = rows * heads_q * HEAD_DIM * 4
    if num_splits <= 1:
        args.num_splits = 1
        args.partial_out = local.data_ptr()
        args.partial_lse = local.data_ptr() + lse_offset
        bdfp4.decode(args, stream)
    else:
        partial_out, partial_lse = ws["partial_out"], ws["partial_lse"]
        args.num_splits = num_splits
        args.bf16_split = 0
        args.out = None
        args.partial_out, args.partial_lse = partial_out.data_ptr(), partial_lse.data_ptr()
        bdfp4.decode(args, stream)
        bdfp4.combine_record(partial_out, partial_lse, num_splits, rows, heads_q, local.data_ptr(),
                             local.data_ptr() + lse_offset, stream)
    dist.all_gather_into_tensor(gathered, local, group=group)
    if out is None:
        out = torch.empty(rows, heads_q, head_dim, dtype=torch.bfloat16, device=device)
    bdfp4.combine_strided(gathered.data_ptr(), record, gathered.data_ptr() + rows * heads_q * HEAD_DIM * 4, record,
                          world, rows, heads_q, out, out.stride(0), stream)
    return out
