"""KV-axis sharding of one long sequence: shard partials from ``bdfp4_decode`` (``out = NULL``),
``[O | LSE]`` records, ``bdfp4_combine_strided``. On one GPU the shards run one after another and
their records are laid out as an all-gather would leave them; with two or more GPUs the same path
runs as NCCL ranks (one process per GPU) through ``bdfp4.distributed.decode_kv_sharded``."""

import os
import sys
from pathlib import Path

import pytest
import torch

from oracle import nvfp4_oracle as oracle

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _shard_args(w, rank, world):
    """Local cache view of ``rank``: its page range through a local page table; rank 0 owns the
    sink, the last rank the rolling tail."""
    from bdfp4.distributed import shard_pages

    pages = int(w.seqused_fp4[0]) // 128
    first, last = shard_pages(pages, world, rank)
    table = w.page_table[:, first:last].contiguous()
    if table.shape[1] == 0:
        table = torch.zeros(w.rows, 1, dtype=torch.int32, device=w.device)
    used = torch.full((w.rows,), (last - first) * 128, dtype=torch.int32, device=w.device)
    residual = w.seqused_residual if rank == world - 1 else torch.zeros_like(w.seqused_residual)
    sink = w.seqused_sink if rank == 0 else torch.zeros_like(w.seqused_sink)
    return table, used, residual, sink, (first, last)


def _oracle_sharded(w, world, splits=1):
    """Every rank's shard decoded by the oracle (split again into ``splits`` parts inside the rank, as
    the CUDA path is asked to), all partials merged at once: a two-level merge is the same sum."""
    from tests.test_gpu_decode import _cpu_cache

    kc, ks, vc, vs = _cpu_cache(w)
    q = oracle.quantize_query(w.query.cpu(), w.heads_kv, terms=2)
    outs, lses = [], []
    for rank in range(world):
        table, used, residual, sink, _ = _shard_args(w, rank, world)
        _, partial, lse = oracle.decode_reference(
            query_values=q["values"], query_padded=q["padded"], key_codes=kc, key_scales=ks, value_codes=vc,
            value_scales=vs, page_table=table.cpu(), seqused_fp4=used.cpu(), heads_kv=w.heads_kv,
            softmax_scale=128 ** -0.5, tail_key=w.tail_key[0].cpu(), tail_value=w.tail_value[0].cpu(),
            tail_slot_ids=w.slot_ids.cpu(), seqused_residual=residual.cpu(), seqused_sink=sink.cpu(),
            num_splits=splits)
        outs.extend(partial)
        lses.extend(lse)
    return oracle.combine_partials(torch.stack(outs), torch.stack(lses))


def _check(got, want):
    err = (got.float().cpu() - want.float()).abs()
    assert float(err.max()) <= 1e-2
    assert float(err.mean() / want.float().abs().mean()) <= 1e-3


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shards_on_one_gpu(world):
    import bdfp4
    from bdfp4.distributed import record_floats
    from bdfp4.workload import build_workload
    from nvfp4_decode_kernel import _decode
    from nvfp4_decode_kernel._quantize import quantize_query

    w = build_workload(rows=1, heads_q=8, heads_kv=2, seq_lens=[2500], sink_tokens=16, seed=5 + world)
    rows, hq = w.rows, w.heads_q
    padded = torch.zeros(rows, 128, hq, 128, dtype=torch.bfloat16, device="cuda")
    quantized = quantize_query(w.query, query_padded_out=padded, heads_kv=w.heads_kv, query_terms=2)
    record = record_floats(rows, hq)
    gathered = torch.full((world * record,), float("nan"), device="cuda")
    stream = bdfp4.current_stream(w.device)
    for rank in range(world):
        table, used, residual, sink, _ = _shard_args(w, rank, world)
        a = bdfp4.DecodeArgs()
        _decode._fill_args(
            a, rows=rows, heads_q=hq, heads_kv=w.heads_kv, page_count=w.regions[0].shape[0],
            query_fp4=quantized[0], query_scales=quantized[1], query_fp4_second=quantized[2],
            query_scales_second=quantized[3], query_padded_bf16=padded, key_pages_fp4=w.regions[0],
            key_scales=w.regions[1], value_pages_fp4=w.regions[2], value_scales=w.regions[3],
            fp4_page_table=table, seqused_fp4=used, residual_key_pages_bf16=w.tail_key[0],
            residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids, seqused_residual=residual,
            seqused_sink=sink, softmax_scale=128 ** -0.5)
        a.num_splits = 1  # out stays NULL: the part leaves as a partial + LSE
        a.partial_out = gathered.data_ptr() + rank * record * 4
        a.partial_lse = a.partial_out + rows * hq * 128 * 4
        bdfp4.decode(a, stream)
    out = torch.empty(rows, hq, 128, dtype=torch.bfloat16, device="cuda")
    bdfp4.combine_strided(gathered.data_ptr(), record, gathered.data_ptr() + rows * hq * 128 * 4, record, world,
                          rows, hq, out, out.stride(0), stream)
    torch.cuda.synchronize()
    _check(out, _oracle_sharded(w, world))


@pytest.mark.parametrize("splits", [3, 7])
def test_shards_split_again_inside_a_rank(splits):
    """A rank's shard is itself split along KV; its parts are folded into the rank's one record by
    bdfp4_combine_record before the (here emulated) exchange."""
    import bdfp4
    from bdfp4.distributed import record_floats
    from bdfp4.workload import build_workload
    from nvfp4_decode_kernel import _decode
    from nvfp4_decode_kernel._quantize import quantize_query

    world = 2
    w = build_workload(rows=1, heads_q=8, heads_kv=2, seq_lens=[4100], sink_tokens=16, seed=15 + splits)
    rows, hq = w.rows, w.heads_q
    padded = torch.zeros(rows, 128, hq, 128, dtype=torch.bfloat16, device="cuda")
    quantized = quantize_query(w.query, query_padded_out=padded, heads_kv=w.heads_kv, query_terms=2)
    record = record_floats(rows, hq)
    gathered = torch.full((world * record,), float("nan"), device="cuda")
    stream = bdfp4.current_stream(w.device)
    for rank in range(world):
        table, used, residual, sink, _ = _shard_args(w, rank, world)
        partial_out = torch.full((splits, rows, hq, 128), float("nan"), device="cuda")
        partial_lse = torch.full((splits, rows, hq), float("nan"), device="cuda")
        a = bdfp4.DecodeArgs()
        _decode._fill_args(
            a, rows=rows, heads_q=hq, heads_kv=w.heads_kv, page_count=w.regions[0].shape[0],
            query_fp4=quantized[0], query_scales=quantized[1], query_fp4_second=quantized[2],
            query_scales_second=quantized[3], query_padded_bf16=padded, key_pages_fp4=w.regions[0],
            key_scales=w.regions[1], value_pages_fp4=w.regions[2], value_scales=w.regions[3],
            fp4_page_table=table, seqused_fp4=used, residual_key_pages_bf16=w.tail_key[0],
            residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids, seqused_residual=residual,
            seqused_sink=sink, softmax_scale=128 ** -0.5)
        a.num_splits = splits
        a.partial_out, a.partial_lse = partial_out.data_ptr(), partial_lse.data_ptr()
        bdfp4.decode(a, stream)
        slot = gathered.data_ptr() + rank * record * 4
        bdfp4.combine_record(partial_out, partial_lse, splits, rows, hq, slot, slot + rows * hq * 128 * 4, stream)
    out = torch.empty(rows, hq, 128, dtype=torch.bfloat16, device="cuda")
    bdfp4.combine_strided(gathered.data_ptr(), record, gathered.data_ptr() + rows * hq * 128 * 4, record, world,
                          rows, hq, out, out.stride(0), stream)
    torch.cuda.synchronize()
    assert not torch.isnan(gathered).any()
    _check(out, _oracle_sharded(w, world, splits))


def _nccl_worker(rank, world, port, result_dir):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "bitdecoding-fp4_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from bdfp4.distributed import decode_kv_sharded
    from bdfp4.workload import build_workload

    # every rank builds the same sequence (same seed); a real deployment holds only its shard
    w = build_workload(rows=1, heads_q=8, heads_kv=2, seq_lens=[2500], sink_tokens=16, seed=77,
                       device=f"cuda:{rank}")
    table, used, residual, sink, _ = _shard_args(w, rank, world)
    out = decode_kv_sharded(
        w.query, *w.regions, table, used, residual_key_pages_bf16=w.tail_key[0],
        residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids, seqused_residual=residual,
        seqused_sink=sink, query_terms=2, num_splits=3)
    torch.cuda.synchronize()
    torch.save(out.cpu(), os.path.join(result_dir, f"out{rank}.pt"))
    if rank == 0:
        torch.save(_oracle_sharded(w, world, 3), os.path.join(result_dir, "want.pt"))
    # the same exchange as ONE kernel over peer memory: identical bits, on every one of several steps
    # (the two record sets alternate), with the rank's parts folded in the kernel and without parts
    from bdfp4.distributed import KvShardedDecoder

    same = True
    for splits in (3, 1):
        kwargs = dict(heads_q=8, rows=1, residual_key_pages_bf16=w.tail_key[0], residual_value_pages_bf16=w.tail_value[0],
                      residual_page_ids=w.slot_ids, seqused_residual=residual, seqused_sink=sink, query_terms=2,
                      num_splits=splits)
        through_nccl = KvShardedDecoder(*w.regions, table, used, **kwargs)(w.query).clone()
        peer = KvShardedDecoder(*w.regions, table, used, exchange="peer", **kwargs)
        for _ in range(5):
            got = peer(w.query)
            torch.cuda.synchronize()
            same = same and torch.equal(got, through_nccl) and int(peer.error.item()) == 0
        dist.barrier()
        peer.close()
    torch.save(torch.tensor(same), os.path.join(result_dir, f"peer_same{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_shards_as_nccl_ranks(tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    port = 29600 + (os.getpid() % 2000)
    mp.start_processes(_nccl_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True,
                       start_method="spawn")
    want = torch.load(tmp_path / "want.pt")
    outs = [torch.load(tmp_path / f"out{r}.pt") for r in range(world)]
    for out in outs:
        _check(out, want)
        assert torch.equal(out, outs[0])  # every rank merges the same records in the same order
    assert all(bool(torch.load(tmp_path / f"peer_same{r}.pt")) for r in range(world))


def test_exchange_kernel_alone_on_one_rank():
    """`bdfp4_exchange_merge` with a world of one (its own region only, nothing to wait for): the fold and
    the merge give the bits of `bdfp4_combine` on the same partials, step after step; argument checks."""
    import bdfp4

    torch.manual_seed(5)
    parts, rows, hq = 3, 2, 8
    partial_out = torch.randn(parts, rows, hq, 128, device="cuda")
    partial_lse = torch.randn(parts, rows, hq, device="cuda") * 3
    partial_lse[1, 0, 3] = float("-inf")  # a part that saw no token
    want = torch.empty(rows, hq, 128, dtype=torch.bfloat16, device="cuda")
    stream = bdfp4.current_stream(want.device)
    bdfp4.combine(partial_out, partial_lse, parts, rows, hq, want, want.stride(0), stream)
    region, _ = bdfp4.peer_alloc(bdfp4.exchange_bytes(1, rows, hq))
    try:
        got = torch.zeros_like(want)
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        a = bdfp4.ExchangeArgs()
        a.partial_out, a.partial_lse, a.parts = partial_out.data_ptr(), partial_lse.data_ptr(), parts
        a.rows, a.heads_q, a.world, a.rank = rows, hq, 1, 0
        a.regions[0] = region
        a.out, a.out_row_stride, a.error_word = got.data_ptr(), got.stride(0), error.data_ptr()
        for step in (1, 2, 3):
            got.zero_()
            a.step = step
            bdfp4.exchange_merge(a, stream)
            torch.cuda.synchronize()
            assert int(error.item()) == 0
            # folding first and merging one record is the merge of the parts up to FP32 rounding of
            # the record: compare in BF16 with one ulp of slack
            assert torch.allclose(got.float(), want.float(), rtol=2 ** -7, atol=1e-6)
        a.step = 0
        with pytest.raises(bdfp4.KernelError):
            bdfp4.exchange_merge(a, stream)
        a.step, a.world = 4, 9
        with pytest.raises(bdfp4.KernelError):
            bdfp4.exchange_merge(a, stream)
    finally:
        bdfp4.peer_free(region)


def test_exchange_reports_a_rank_that_never_sends():
    """Failure detection without a fault: a world of two in which the other rank takes no part. Its flag
    is never written, so the kernel's bounded wait (two seconds) runs out: it reports
    DEV_WAIT_TIMEOUT in the error word, leaves that rank out of the merge and returns; the context
    stays usable (the next, complete exchange on the same regions gives the right answer)."""
    import bdfp4

    torch.manual_seed(9)
    rows, hq = 1, 8
    partial_out = torch.randn(1, rows, hq, 128, device="cuda")
    partial_lse = torch.randn(1, rows, hq, device="cuda")
    want = torch.empty(rows, hq, 128, dtype=torch.bfloat16, device="cuda")
    stream = bdfp4.current_stream(want.device)
    bdfp4.combine(partial_out, partial_lse, 1, rows, hq, want, want.stride(0), stream)
    size = bdfp4.exchange_bytes(2, rows, hq)
    mine, _ = bdfp4.peer_alloc(size)
    silent, _ = bdfp4.peer_alloc(size)  # stands for the other rank's region; nobody runs as that rank
    try:
        got = torch.zeros_like(want)
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        a = bdfp4.ExchangeArgs()
        a.partial_out, a.partial_lse, a.parts = partial_out.data_ptr(), partial_lse.data_ptr(), 1
        a.rows, a.heads_q, a.world, a.rank, a.step = rows, hq, 2, 0, 1
        a.regions[0], a.regions[1] = mine, silent
        a.out, a.out_row_stride, a.error_word = got.data_ptr(), got.stride(0), error.data_ptr()
        bdfp4.exchange_merge(a, stream)
        torch.cuda.synchronize()
        assert int(error.item()) & bdfp4.DEV_WAIT_TIMEOUT
        assert torch.equal(got, want)  # only this rank's record was merged
        # the context is intact: a world of one (fresh region) completes at once, without a report
        error.zero_()
        got.zero_()
        alone, _ = bdfp4.peer_alloc(bdfp4.exchange_bytes(1, rows, hq))
        a.world, a.step = 1, 2
        a.regions[0] = alone
        bdfp4.exchange_merge(a, stream)
        torch.cuda.synchronize()
        bdfp4.peer_free(alone)
        assert int(error.item()) == 0 and torch.equal(got, want)
    finally:
        bdfp4.peer_free(mine)
        bdfp4.peer_free(silent)
