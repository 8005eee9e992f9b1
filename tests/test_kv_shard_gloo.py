"""The KV-axis shard + one all-gather + merge path on two CPU ranks (gloo): page partition, the
``[O | LSE]`` record exchanged by one all_gather, and the LSE-weighted merge. Each rank computes
its shard's partial with the CPU oracle; the merged result must equal the single-process split of
the same sequence exactly (same arithmetic, same part order)."""

import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
WORLD = 2


def _sequence(seed=11, tokens=1300, heads_q=8, heads_kv=2):
    sys.path.insert(0, str(ROOT))
    from tests.test_oracle_decode import _case

    return _case([tokens], heads_q=heads_q, heads_kv=heads_kv, seed=seed)


def _worker(rank: int, port: int, result_path: str) -> None:
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "bitdecoding-fp4_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    from bdfp4.distributed import record_floats, shard_pages, split_record
    from oracle import nvfp4_oracle as oracle

    q, cache, meta, _ = _sequence()
    kc, ks, vc, vs = cache
    rows, heads_q = q.shape[0], q.shape[1]
    pages = int(meta["seqused_fp4"][0]) // 128
    first, last = shard_pages(pages, WORLD, rank)
    # this rank's shard: its own pages through a local page table; rank 0 owns the sink, the last
    # rank the rolling tail
    local = dict(meta)
    local["page_table"] = meta["page_table"][:, first:last].contiguous()
    local["seqused_fp4"] = torch.tensor([(last - first) * 128], dtype=torch.int32)
    local["seqused_residual"] = meta["seqused_residual"] if rank == WORLD - 1 else torch.zeros(1, dtype=torch.int32)
    local["seqused_sink"] = meta["seqused_sink"] if rank == 0 else torch.zeros(1, dtype=torch.int32)
    qq = oracle.quantize_query(q, 2, terms=2)
    _, partial, lse = oracle.decode_reference(
        query_values=qq["values"], query_padded=qq["padded"], key_codes=kc, key_scales=ks, value_codes=vc,
        value_scales=vs, heads_kv=2, softmax_scale=128 ** -0.5, **local)
    record = torch.cat([partial[0].reshape(-1), lse[0].reshape(-1)])
    assert record.numel() == record_floats(rows, heads_q)
    gathered = torch.empty(WORLD * record.numel())
    dist.all_gather_into_tensor(gathered, record)  # the one exchange of the path
    outs, lses = split_record(gathered, WORLD, rows, heads_q)
    merged = oracle.combine_partials(outs, lses)
    if rank == 0:
        torch.save({"merged": merged, "outs": outs.clone(), "lses": lses.clone()}, result_path)
    dist.barrier()
    dist.destroy_process_group()


def test_shard_pages_partition():
    sys.path.insert(0, str(ROOT / "bitdecoding-fp4_b200"))
    from bdfp4.distributed import shard_pages

    for total in (0, 1, 7, 8, 8191):
        for world in (1, 2, 4, 8):
            ranges = [shard_pages(total, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            assert max(b - a for a, b in ranges) <= -(-total // world) if total else True
    with pytest.raises(ValueError):
        shard_pages(8, 2, 2)


@pytest.mark.timeout(300)
def test_two_rank_kv_shard_merge_matches_single_process(tmp_path):
    from oracle import nvfp4_oracle as oracle

    result = tmp_path / "merged.pt"
    port = 29500 + (os.getpid() % 2000)
    mp.start_processes(_worker, args=(port, str(result)), nprocs=WORLD, join=True, start_method="spawn")
    got = torch.load(result)
    q, cache, meta, sources = _sequence()
    kc, ks, vc, vs = cache
    qq = oracle.quantize_query(q, 2, terms=2)
    # every shard here masks against its own running maximum, exactly like an intra-GPU split
    whole, _, _ = oracle.decode_reference(
        query_values=qq["values"], query_padded=qq["padded"], key_codes=kc, key_scales=ks, value_codes=vc,
        value_scales=vs, heads_kv=2, softmax_scale=128 ** -0.5, **meta)
    err = (got["merged"].float() - whole.float()).abs()
    assert float(err.mean() / whole.float().abs().mean()) < 0.1  # FP4-P noise between partitions
    k, v = sources[0]
    for h in range(2):
        plain = oracle.plain_attention(q[0, 4 * h:4 * h + 4], k[:, h], v[:, h], 128 ** -0.5)
        rel = ((got["merged"][0, 4 * h:4 * h + 4].float() - plain).abs().mean() / plain.abs().mean()).item()
        assert rel < 0.25
    assert torch.isfinite(got["lses"]).all()
