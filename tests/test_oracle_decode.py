"""CPU-only consistency checks of the oracle's whole-batch decode (the checker of the GPU tests)."""

import torch

from oracle import nvfp4_oracle as oracle


def _case(seq_lens, heads_q=8, heads_kv=2, seed=0, sink=16):
    gen = torch.Generator().manual_seed(seed)
    rows = len(seq_lens)
    pages_per_row = [oracle.split_sequence_length(n, sink)[1] // 128 for n in seq_lens]
    blocks = 1 + sum(pages_per_row)
    kc = torch.zeros(blocks, 128, heads_kv, 64, dtype=torch.uint8)
    ks = torch.zeros(blocks, heads_kv, 1024, dtype=torch.uint8)
    vc = torch.zeros(blocks, heads_kv, 128, 64, dtype=torch.uint8)
    vs = torch.zeros(blocks, heads_kv, 1024, dtype=torch.uint8)
    table = torch.zeros(rows, max(1, max(pages_per_row)), dtype=torch.int32)
    tail_k = torch.zeros(rows, 144, heads_kv, 128, dtype=torch.bfloat16)
    tail_v = torch.zeros_like(tail_k)
    order = torch.randperm(blocks - 1, generator=gen) + 1
    cursor, sources = 0, []
    for row, n in enumerate(seq_lens):
        s, fp4, tail = oracle.split_sequence_length(n, sink)
        k = torch.randn(n, heads_kv, 128, generator=gen).to(torch.bfloat16)
        v = torch.randn(n, heads_kv, 128, generator=gen).to(torch.bfloat16)
        pages = fp4 // 128
        ids = order[cursor:cursor + pages]
        cursor += pages
        table[row, :pages] = ids.int()
        if pages:
            kc[ids], ks[ids] = oracle.quantize_key_pages(k[:fp4].reshape(pages, 128, heads_kv, 128))
            vc[ids], vs[ids] = oracle.quantize_value_pages(v[:fp4].reshape(pages, 128, heads_kv, 128))
        tail_k[row, :tail], tail_v[row, :tail] = k[fp4:], v[fp4:]
        tail_k[row, 128:128 + s], tail_v[row, 128:128 + s] = k[:s], v[:s]
        sources.append((k, v))
    q = torch.randn(rows, heads_q, 128, generator=gen).to(torch.bfloat16)
    lens = [oracle.split_sequence_length(n, sink) for n in seq_lens]
    meta = dict(
        page_table=table, seqused_fp4=torch.tensor([x[1] for x in lens], dtype=torch.int32),
        tail_key=tail_k, tail_value=tail_v, tail_slot_ids=torch.arange(rows, dtype=torch.int32),
        seqused_residual=torch.tensor([x[2] for x in lens], dtype=torch.int32),
        seqused_sink=torch.tensor([x[0] for x in lens], dtype=torch.int32),
    )
    return q, (kc, ks, vc, vs), meta, sources


def _run(q, cache, meta, heads_kv=2, terms=2, **kw):
    qq = oracle.quantize_query(q, heads_kv, terms=terms)
    kc, ks, vc, vs = cache
    return oracle.decode_reference(
        query_values=qq["values"], query_padded=qq["padded"], key_codes=kc, key_scales=ks, value_codes=vc,
        value_scales=vs, heads_kv=heads_kv, softmax_scale=128 ** -0.5, **meta, **kw)


def test_decode_reference_close_to_plain_attention():
    q, cache, meta, sources = _case([300, 100, 1, 513])
    out, _, _ = _run(q, cache, meta)
    for row, (k, v) in enumerate(sources):
        for h in range(2):
            want = oracle.plain_attention(q[row, 4 * h:4 * h + 4], k[:, h], v[:, h], 128 ** -0.5)
            got = out[row, 4 * h:4 * h + 4].float()
            rel = ((got - want).abs().mean() / want.abs().mean()).item()
            assert rel < 0.25, (row, h, rel)
    # rows with no FP4 page are BF16 throughout: only rounding separates them from the plain result
    want = oracle.plain_attention(q[2, :4], sources[2][0][:, 0], sources[2][1][:, 0], 128 ** -0.5)
    torch.testing.assert_close(out[2, :4].float(), want, rtol=2e-2, atol=2e-2)


def test_split_merge_matches_unsplit():
    q, cache, meta, _ = _case([900, 257], seed=3)
    whole, _, _ = _run(q, cache, meta)
    for splits, own in ((2, False), (3, True), (8, True)):
        merged, partial, lse = _run(q, cache, meta, num_splits=splits, bf16_split=own)
        assert partial.shape[0] == splits + int(own)
        err = (merged.float() - whole.float()).abs()
        # each part quantises P against its own running maximum, so parts differ by FP4-P noise
        assert float(err.max()) < 5e-2 and float(err.mean() / whole.float().abs().mean()) < 0.1


def test_rows_without_slot_or_pages():
    q, cache, meta, _ = _case([200, 64], seed=5)
    meta["tail_slot_ids"][0] = -1
    out, _, lse = _run(q, cache, meta, terms=1)
    assert torch.isfinite(out.float()).all()
    meta["seqused_fp4"][:] = 0
    out, _, lse = _run(q, cache, meta, terms=1)
    assert float(out[0].float().abs().sum()) == 0.0 and bool(torch.isinf(lse[0, 0]).all())
