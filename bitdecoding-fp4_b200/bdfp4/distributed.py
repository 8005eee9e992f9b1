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


class PeerExchange:
    """The exchange regions of a process group's ranks on one node, for ``bdfp4_exchange_merge``: this
    rank's region (allocated by the library, zeroed) and every other rank's mapped into this process
    through CUDA IPC. Building one is a collective call (the 64-byte handles travel by
    ``all_gather_object``) and allocates: set-up only. ``close()`` unmaps and frees; call it on every
    rank before the process group goes away."""

    def __init__(self, rows: int, heads_q: int, group=None):
        import torch.distributed as dist

        import bdfp4

        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.rows, self.heads_q = rows, heads_q
        self.bytes = bdfp4.exchange_bytes(self.world, rows, heads_q)
        self.local, handle = bdfp4.peer_alloc(self.bytes)
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        self.regions = [self.local if r == self.rank else bdfp4.peer_open(handles[r]) for r in range(self.world)]
        self.step = 0
        dist.barrier(group)  # nobody stores into a region before everyone has mapped it

    def next_step(self) -> int:
        """The stamp of the next exchange: 1, 2, ... (never 0), the same on every rank."""
        self.step = self.step % 0xFFFFFFFF + 1
        return self.step

    def close(self) -> None:
        import bdfp4

        for r, address in enumerate(self.regions):
            if r != self.rank:
                bdfp4.peer_close(address)
        bdfp4.peer_free(self.local)
        self.regions = []


class KvShardedDecoder:
    """One rank's side of the KV-sharded decode, with everything that does not change between steps held
    across them: the shard's cache regions and metadata, the two argument records of the C ABI, the query
    quantizer's outputs, the split partials, the rank's ``[O | LSE]`` record and the gathered records.

    A step is :meth:`__call__` with the step's query: it writes the query's address into the records and
    issues the launches back to back on torch's current stream, with no allocation, no validation of
    device values and no host synchronisation: query quantizer, shard decode (split again inside the rank
    when ``num_splits > 1``), fold of the rank's parts into its record, ONE ``all_gather`` of the records,
    merge. This library's kernels are launched with programmatic stream serialization, so each one's CTAs
    come up while its predecessor drains.

    With ``exchange="peer"`` (ranks of one node, one process per GPU) the last three are ONE launch,
    ``bdfp4_exchange_merge``: each rank stores its record straight into the other ranks' memory over
    NVLink and merges what arrives in its own; same results, bit for bit. Call :meth:`close` at the end.

    Pass the BF16 residual arguments only on the rank that owns them (see the module docstring); with
    ``seqused_sink`` but ``seqused_residual`` zero a rank owns the sink alone.
    """

    def __init__(self, key_pages_fp4, key_scales, value_pages_fp4, value_scales, fp4_page_table, seqused_fp4, *,
                 heads_q: int, rows: int = 1, group=None, residual_key_pages_bf16=None,
                 residual_value_pages_bf16=None, residual_page_ids=None, seqused_residual=None, seqused_sink=None,
                 softmax_scale: float | None = None, query_terms: int = 2, scale_mode: str = "amax6",
                 query_rotation: str = "none", out: torch.Tensor | None = None, num_splits: int | None = None,
                 exchange: str = "nccl"):
        import torch.distributed as dist

        import bdfp4
        from nvfp4_decode_kernel import _decode
        from nvfp4_decode_kernel.scale_mode import mode_id

        self.group, self.world = group, dist.get_world_size(group)
        self.rows, self.heads_q = rows, heads_q
        heads_kv = key_pages_fp4.shape[2]
        device = key_pages_fp4.device
        self.device = device
        has_residual = residual_key_pages_bf16 is not None
        if num_splits is None:
            # a shard of one sequence is only `heads_kv` walks: cut it until the launch fills the GPU at four
            # CTAs per SM (the default cap of 32 parts would leave one or two CTAs per SM here)
            num_splits = _decode.resident_num_splits(rows, heads_kv, sms=_decode._multiprocessor_count(device.index or 0),
                                                     max_splits=128)
        self.num_splits = num_splits
        self.record = record_floats(rows, heads_q)
        # buffers: whatever the per-call form would allocate
        u8 = dict(dtype=torch.uint8, device=device)
        self.codes = [torch.zeros(rows, 1, heads_q, HEAD_DIM // 2, **u8) for _ in range(query_terms)]
        self.scales = [torch.zeros(rows, 1, heads_q, 2, 32, 4, 4, **u8) for _ in range(query_terms)]
        # rows past the first of each padded query tile stay zero: written once, here
        self.padded = torch.zeros(rows, 128, heads_q, HEAD_DIM, dtype=torch.bfloat16, device=device) if has_residual else None
        self.local = torch.empty(self.record, dtype=torch.float32, device=device)
        self.gathered = torch.empty(self.world * self.record, dtype=torch.float32, device=device)
        self.out = out if out is not None else torch.empty(rows, heads_q, HEAD_DIM, dtype=torch.bfloat16, device=device)
        self.partial_out = self.partial_lse = None
        if num_splits > 1:
            self.partial_out = torch.empty(num_splits, rows, heads_q, HEAD_DIM, dtype=torch.float32, device=device)
            self.partial_lse = torch.empty(num_splits, rows, heads_q, dtype=torch.float32, device=device)
        # the quantizer's record: only `query` changes between steps
        q = bdfp4.QuantizeQueryArgs()
        q.rows, q.heads_q, q.heads_kv = rows, heads_q, heads_kv
        q.scale_mode, q.rotate = mode_id(scale_mode), int(query_rotation == "hadamard")
        q.query_codes, q.query_scales = self.codes[0].data_ptr(), self.scales[0].data_ptr()
        if query_terms == 2:
            q.query_codes_second, q.query_scales_second = self.codes[1].data_ptr(), self.scales[1].data_ptr()
        q.query_padded = bdfp4.ptr(self.padded)
        self.quantize_args = q
        # the decode record: nothing changes between steps (lengths and tables are read on the device)
        from nvfp4_decode_kernel._quantize import _scale_view

        a = bdfp4.DecodeArgs()
        views = [_scale_view(s, heads_kv) for s in self.scales]
        _decode._fill_args(
            a, rows=rows, heads_q=heads_q, heads_kv=heads_kv, page_count=key_pages_fp4.shape[0],
            query_fp4=self.codes[0], query_scales=views[0], query_fp4_second=self.codes[1] if query_terms == 2 else None,
            query_scales_second=views[1] if query_terms == 2 else None, query_padded_bf16=self.padded,
            key_pages_fp4=key_pages_fp4, key_scales=key_scales, value_pages_fp4=value_pages_fp4,
            value_scales=value_scales, fp4_page_table=fp4_page_table, seqused_fp4=seqused_fp4,
            residual_key_pages_bf16=residual_key_pages_bf16, residual_value_pages_bf16=residual_value_pages_bf16,
            residual_page_ids=residual_page_ids, seqused_residual=seqused_residual, seqused_sink=seqused_sink,
            softmax_scale=softmax_scale if softmax_scale is not None else HEAD_DIM ** -0.5)
        self.lse_offset = rows * heads_q * HEAD_DIM * 4
        if num_splits <= 1:
            a.num_splits = 1
            a.partial_out, a.partial_lse = self.local.data_ptr(), self.local.data_ptr() + self.lse_offset
        else:
            a.num_splits, a.bf16_split, a.out = num_splits, 0, None
            a.partial_out, a.partial_lse = self.partial_out.data_ptr(), self.partial_lse.data_ptr()
        self.decode_args = a
        # exchange="peer": fold, exchange and merge are ONE kernel storing into the peers' memory
        # (bdfp4_exchange_merge) instead of fold kernel + NCCL all-gather + merge kernel
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        self.peers = None
        if exchange == "peer":
            self.peers = PeerExchange(rows, heads_q, group)
            x = bdfp4.ExchangeArgs()
            x.rows, x.heads_q, x.world, x.rank = rows, heads_q, self.world, self.peers.rank
            if num_splits > 1:
                x.partial_out, x.partial_lse, x.parts = self.partial_out.data_ptr(), self.partial_lse.data_ptr(), num_splits
            else:
                x.partial_out, x.partial_lse, x.parts = self.local.data_ptr(), self.local.data_ptr() + self.lse_offset, 1
            for r, address in enumerate(self.peers.regions):
                x.regions[r] = address
            x.out, x.out_row_stride = self.out.data_ptr(), self.out.stride(0)
            self.error = torch.zeros(1, dtype=torch.int32, device=device)
            x.error_word = self.error.data_ptr()
            self.exchange_args = x
        self._keep = (key_pages_fp4, key_scales, value_pages_fp4, value_scales, fp4_page_table, seqused_fp4,
                      residual_key_pages_bf16, residual_value_pages_bf16, residual_page_ids, seqused_residual,
                      seqused_sink)  # the records hold raw addresses: keep their owners alive

    def __call__(self, query: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        import bdfp4

        if query.dtype is not torch.bfloat16 or tuple(query.shape) != (self.rows, self.heads_q, HEAD_DIM) \
                or query.stride(-1) != 1 or query.data_ptr() % 16 or query.stride(0) % 8 or query.stride(1) % 8:
            raise ValueError(f"query must be BF16 [{self.rows}, {self.heads_q}, {HEAD_DIM}] with 16-byte aligned heads")
        q = self.quantize_args
        q.query, q.query_row_stride, q.query_head_stride = query.data_ptr(), query.stride(0), query.stride(1)
        stream = bdfp4.current_stream(self.device)
        bdfp4.quantize_query(q, stream)
        bdfp4.decode(self.decode_args, stream)
        if self.peers is not None:
            self.exchange_args.step = self.peers.next_step()
            bdfp4.exchange_merge(self.exchange_args, stream)
            return self.out
        if self.num_splits > 1:
            bdfp4.combine_record(self.partial_out, self.partial_lse, self.num_splits, self.rows, self.heads_q,
                                 self.local.data_ptr(), self.local.data_ptr() + self.lse_offset, stream)
        dist.all_gather_into_tensor(self.gathered, self.local, group=self.group)
        bdfp4.combine_strided(self.gathered.data_ptr(), self.record, self.gathered.data_ptr() + self.lse_offset,
                              self.record, self.world, self.rows, self.heads_q, self.out, self.out.stride(0), stream)
        return self.out


    def close(self) -> None:
        """Release the peer mappings (a collective-free call, but make it on every rank)."""
        if self.peers is not None:
            self.peers.close()
            self.peers = None


def decode_kv_sharded(query: torch.Tensor, key_pages_fp4, key_scales, value_pages_fp4, value_scales,
                      fp4_page_table: torch.Tensor, seqused_fp4: torch.Tensor, *, group=None,
                      residual_key_pages_bf16=None, residual_value_pages_bf16=None, residual_page_ids=None,
                      seqused_residual=None, seqused_sink=None, softmax_scale: float | None = None,
                      query_terms: int = 2, scale_mode: str = "amax6", query_rotation: str = "none",
                      out: torch.Tensor | None = None, num_splits: int | None = None,
                      workspace: dict | None = None) -> torch.Tensor:
    """Decode attention over a sequence whose FP4 pages are sharded across the ranks of ``group``: the
    one-call form of :class:`KvShardedDecoder`. Every rank passes the same ``query`` and its own shard.
    ``workspace`` (a dict the caller keeps between steps) holds the decoder, so that only the first call
    builds it; it is tied to the tensors of that first call. Returns the merged BF16 output on every rank."""
    rows, heads_q, _ = query.shape
    ws = workspace if workspace is not None else {}
    key = (rows, heads_q, key_pages_fp4.data_ptr(), fp4_page_table.data_ptr(), seqused_fp4.data_ptr(),
           residual_key_pages_bf16 is not None, None if seqused_residual is None else seqused_residual.data_ptr(),
           None if seqused_sink is None else seqused_sink.data_ptr(), num_splits, query_terms, scale_mode,
           query_rotation, None if out is None else out.data_ptr())
    if ws.get("key") != key:
        ws.clear()
        ws["key"] = key
        ws["decoder"] = KvShardedDecoder(
            key_pages_fp4, key_scales, value_pages_fp4, value_scales, fp4_page_table, seqused_fp4, heads_q=heads_q,
            rows=rows, group=group, residual_key_pages_bf16=residual_key_pages_bf16,
            residual_value_pages_bf16=residual_value_pages_bf16, residual_page_ids=residual_page_ids,
            seqused_residual=seqused_residual, seqused_sink=seqused_sink, softmax_scale=softmax_scale,
            query_terms=query_terms, scale_mode=scale_mode, query_rotation=query_rotation, out=out,
            num_splits=num_splits)
    return ws["decoder"](query)
