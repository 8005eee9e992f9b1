"""Paged FP4 decode attention (through the package API and the C ABI) against the CPU oracle.

Tolerance: max |err| <= 1e-2 and mean relative error <= 1e-3, both in BF16, against the oracle
that models the kernel's own operands (FP4 query terms, FP4 probabilities, block order,
stale-maximum rule). The kernel uses ex2.approx / rcp.approx, so agreement is statistical rather
than bitwise.
"""

import math

import pytest
import torch

from oracle import nvfp4_oracle as oracle

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_REL = 1e-2, 1e-3


def _scale_tiles(blocks_cpu, heads, offset):
    """[blocks, H, 1024] scale bytes of the region starting at ``offset`` of each flat block."""
    return blocks_cpu[:, offset:offset + heads * 1024].reshape(-1, heads, 1024)


def _cpu_cache(w):
    blocks = w.blocks.cpu()
    h = w.heads_kv
    key_codes = blocks[:, :8192 * h].reshape(-1, 128, h, 64)
    key_scales = _scale_tiles(blocks, h, 8192 * h)
    value_codes = blocks[:, 9216 * h:17408 * h].reshape(-1, h, 128, 64)
    value_scales = _scale_tiles(blocks, h, 17408 * h)
    return key_codes, key_scales, value_codes, value_scales


def _oracle_decode(w, *, terms, scale_mode, rotate, num_splits=1, bf16_split=False, with_tail=True,
                   p_mode="amax2_or_amax6_c8", bf16_page_cost=0, tau=oracle.DEFAULT_P_TAU, query_scale=1.0):
    kc, ks, vc, vs = _cpu_cache(w)
    q = oracle.quantize_query(w.query.cpu(), w.heads_kv, scale_mode=scale_mode, terms=terms, rotate=rotate,
                              tensor_scale=query_scale)
    kwargs = {}
    if with_tail:
        kwargs = dict(tail_key=w.tail_key[0].cpu(), tail_value=w.tail_value[0].cpu(),
                      tail_slot_ids=w.slot_ids.cpu(), seqused_residual=w.seqused_residual.cpu(),
                      seqused_sink=w.seqused_sink.cpu() if w.sink_tokens else None)
    return oracle.decode_reference(
        query_values=q["values"], query_padded=q["padded"], key_codes=kc, key_scales=ks, value_codes=vc,
        value_scales=vs, page_table=w.page_table.cpu(), seqused_fp4=w.seqused_fp4.cpu(), heads_kv=w.heads_kv,
        softmax_scale=128 ** -0.5, p_mode=p_mode, tau=tau, num_splits=num_splits, bf16_split=bf16_split,
        bf16_page_cost=bf16_page_cost, tensor_scales=(w.tensor_scales[0], query_scale, w.tensor_scales[2]),
        **kwargs)


def _check(got, want, label="", large_outputs=False):
    """``large_outputs``: the absolute bound scales with |value| above 1. Where attention concentrates
    on a few tokens the outputs reach 2-4, and one BF16 step there (2^-6) already exceeds 1e-2."""
    got, want = got.float().cpu(), want.float()
    assert torch.isfinite(got).all(), label
    err = (got - want).abs()
    mean_rel = float(err.mean() / want.abs().mean().clamp_min(1e-12))
    bound = MAX_ABS * want.abs().clamp_min(1.0) if large_outputs else torch.full_like(err, MAX_ABS)
    assert bool((err <= bound).all()), f"{label} max abs err {float(err.max()):.3e}"
    assert mean_rel <= MEAN_REL, f"{label} mean rel err {mean_rel:.3e}"
    return float(err.max()), mean_rel


def _decode(w, *, terms=1, scale_mode="amax6", rotate=False, num_splits=1, with_tail=True, **extra):
    from nvfp4_decode_kernel import fp4_decode

    kwargs = dict(extra)
    if with_tail:
        kwargs.update(residual_key_pages_bf16=w.tail_key[0], residual_value_pages_bf16=w.tail_value[0],
                      residual_page_ids=w.slot_ids, seqused_residual=w.seqused_residual)
        if w.sink_tokens:
            kwargs.update(seqused_sink=w.seqused_sink)
    return fp4_decode(w.query, *w.regions, w.page_table, w.seqused_fp4, query_terms=terms,
                      scale_mode=scale_mode, query_rotation="hadamard" if rotate else "none",
                      num_splits=num_splits, **kwargs)


def test_cache_fill_matches_oracle():
    """The workload builder's writer calls: pages land where the block table says, the rolling
    tail and the sink hold the right tokens (K in the cache basis)."""
    from bdfp4.workload import build_workload

    w = build_workload(rows=3, heads_q=8, heads_kv=2, seq_lens=[700, 130, 9], sink_tokens=16, seed=4,
                       key_scale_mode="four_six", value_scale_mode="amax6", rotate=True, key_shift=True,
                       keep_source=True, chunk_pages=2)
    kc, ks, vc, vs = _cpu_cache(w)
    shift = w.key_shift[0].cpu()
    for row, n in enumerate(w.seq_lens):
        k, v = (t.cpu() for t in w.kept[row])
        sink, fp4, tail = oracle.split_sequence_length(n)
        assert (int(w.seqused_fp4[row]), int(w.seqused_residual[row]), int(w.seqused_sink[row])) == (fp4, tail, sink)
        pages = fp4 // 128
        ids = w.page_table[row, :pages].cpu().long()
        if pages:
            want_kc, want_ks = oracle.quantize_key_pages(k[:fp4].reshape(pages, 128, 2, 128), "four_six",
                                                         rotate=True, shift=shift)
            want_vc, want_vs = oracle.quantize_value_pages(v[:fp4].reshape(pages, 128, 2, 128), "amax6")
            assert torch.equal(kc[ids], want_kc) and torch.equal(ks[ids], want_ks)
            assert torch.equal(vc[ids], want_vc) and torch.equal(vs[ids], want_vs)
        basis = oracle.key_cache_basis(k, rotate=True, shift=shift)
        assert torch.equal(w.tail_key[0, row, :tail].cpu(), basis[fp4:n])
        assert torch.equal(w.tail_value[0, row, :tail].cpu(), v[fp4:n])
        assert torch.equal(w.tail_key[0, row, 128:128 + sink].cpu(), basis[:sink])
        assert torch.equal(w.tail_value[0, row, 128:128 + sink].cpu(), v[:sink])


@pytest.mark.parametrize("heads_q,heads_kv", [(8, 2), (16, 2), (32, 2)])
@pytest.mark.parametrize("terms", [1, 2])
def test_decode_pages_only(heads_q, heads_kv, terms):
    """FP4 pages alone (no BF16 residual): 1-5 pages per row, one row with none."""
    from bdfp4.workload import build_workload

    w = build_workload(rows=4, heads_q=heads_q, heads_kv=heads_kv, seq_lens=[641, 129, 385, 100], sink_tokens=0,
                       seed=heads_q + terms)
    out = _decode(w, terms=terms, with_tail=False)
    want, _, _ = _oracle_decode(w, terms=terms, scale_mode="amax6", rotate=False, with_tail=False)
    rows_with_pages = [0, 1, 2]
    _check(out[rows_with_pages], want[rows_with_pages], f"G={heads_q // heads_kv} terms={terms}")
    assert float(out[3].float().abs().sum()) == 0.0  # no FP4 tokens, no residual: nothing attends


@pytest.mark.parametrize("sink_tokens", [16, 4, 0])
def test_decode_small_batch_with_the_serving_recipe(sink_tokens):
    """Batch 4, 8 query / 2 KV heads, contexts uniform in [512, 2048], BF16 sink and rolling tail,
    the recipe the reference serves with (two query terms, Hadamard, four_six K, key shift)."""
    from bdfp4.workload import build_workload

    gen = torch.Generator().manual_seed(0)
    lens = torch.randint(512, 2049, (4,), generator=gen).tolist()
    w = build_workload(rows=4, heads_q=8, heads_kv=2, seq_lens=lens, sink_tokens=sink_tokens, seed=1,
                       key_scale_mode="four_six", rotate=True, key_shift=True)
    if sink_tokens not in (0, 16):
        # the decode entry takes the sink in rows [128, 144) of a 144-row buffer
        pad = torch.zeros(1, 4, 144, 2, 128, dtype=torch.bfloat16, device="cuda")
        pad_v = pad.clone()
        pad[:, :, :128 + sink_tokens] = w.tail_key
        pad_v[:, :, :128 + sink_tokens] = w.tail_value
        w.tail_key, w.tail_value = pad, pad_v
    out = _decode(w, terms=2, scale_mode="four_six", rotate=True)
    want, _, _ = _oracle_decode(w, terms=2, scale_mode="four_six", rotate=True)
    _check(out, want, f"sink={sink_tokens}")


def test_decode_edge_rows():
    """Tail only (no page yet, sink masked inside the rolling page), exactly one full page,
    a row without a tail slot, a one-token sequence."""
    from bdfp4.workload import build_workload

    w = build_workload(rows=5, heads_q=8, heads_kv=2, seq_lens=[100, 128, 129, 1, 300], sink_tokens=16, seed=7)
    w.slot_ids[4] = -1  # a row the control plane gave no slot: only its FP4 pages attend
    with pytest.raises(ValueError):
        _decode(w, terms=1)  # a negative slot id is refused unless the metadata is trusted
    out = _decode(w, terms=1, trusted_metadata=True)
    want, _, _ = _oracle_decode(w, terms=1, scale_mode="amax6", rotate=False)
    _check(out, want, "edge rows")


@pytest.mark.parametrize("num_splits", [2, 3, 8])
def test_decode_split_kv(num_splits):
    from bdfp4.workload import build_workload

    w = build_workload(rows=2, heads_q=8, heads_kv=2, seq_lens=[1500, 260], sink_tokens=16, seed=num_splits)
    out = _decode(w, terms=2, num_splits=num_splits)
    unsplit = _decode(w, terms=2)
    want, _, _ = _oracle_decode(w, terms=2, scale_mode="amax6", rotate=False, num_splits=num_splits,
                                bf16_split=True)
    _check(out, want, f"splits={num_splits}")
    # parts quantise P against their own running maxima: split and unsplit differ by FP4-P noise
    rel = ((out.float() - unsplit.float()).abs().mean() / unsplit.float().abs().mean()).item()
    assert rel < 0.1, rel


@pytest.mark.parametrize("cost", [0, 6])
def test_decode_split_kv_shared_bf16_split(cost, monkeypatch):
    """A launch too wide to give the tail and sink CTAs of their own: split 0 merges them, under the
    even partition and when it is charged `cost` pages for them (rows with fewer pages included)."""
    from bdfp4.workload import build_workload
    from nvfp4_decode_kernel import _decode as decode_module
    from nvfp4_decode_kernel import split_partial_count

    monkeypatch.setattr(decode_module, "BF16_BLOCK_PAGE_COST", cost)
    BF16_BLOCK_PAGE_COST = cost
    rows, splits = 80, 2
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert split_partial_count(rows, 2, splits, residual=True, sms=sms) == splits
    lengths = [131 + 97 * (i % 23) + (2200 if i % 7 == 0 else 0) for i in range(rows)]
    w = build_workload(rows=rows, heads_q=8, heads_kv=2, seq_lens=lengths, sink_tokens=16, seed=31)
    out = _decode(w, terms=2, num_splits=splits)
    want, _, _ = _oracle_decode(w, terms=2, scale_mode="amax6", rotate=False, num_splits=splits,
                                bf16_split=False, bf16_page_cost=BF16_BLOCK_PAGE_COST)
    _check(out, want, f"shared bf16 split, cost {cost}")


@pytest.mark.parametrize("rows,num_splits,page_tokens", [(3, 4, 128), (80, 2, 128), (5, 3, 64)])
def test_decode_fused_split_merge(rows, num_splits, page_tokens):
    """With a counter array the split launch merges its own partials: bit-identical to the separate
    merge kernel (same arithmetic, same part order), counters back at zero, repeatable."""
    from bdfp4.workload import build_workload

    lengths = [150 + 211 * (i % 9) + (1900 if i % 5 == 0 else 0) for i in range(rows)]
    w = build_workload(rows=rows, heads_q=8, heads_kv=2, seq_lens=lengths, sink_tokens=16, seed=rows,
                       page_tokens=page_tokens)
    want = _decode(w, terms=2, num_splits=num_splits).clone()
    counters = torch.zeros(rows * 2 + 7, dtype=torch.int32, device="cuda")
    for _ in range(3):
        out = torch.full((rows, 8, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        got = _decode(w, terms=2, num_splits=num_splits, split_merge_counters=counters, out=out)
        assert torch.equal(got, want)
        assert int(counters.abs().sum()) == 0
    with pytest.raises(ValueError):
        _decode(w, terms=2, num_splits=num_splits, split_merge_counters=counters[:rows])


def test_decode_rows_cut_into_different_numbers_of_parts():
    """`row_splits`: in one launch of four parts a row is cut into its own number of parts; its further
    parts leave with an LSE of -inf. A row cut into k parts gives the bits of a launch with k parts for
    every row (same page ranges, and the merge passes over -inf parts), and agrees with the oracle."""
    from bdfp4.workload import build_workload

    w = build_workload(rows=3, heads_q=8, heads_kv=2, seq_lens=[2300, 700, 1500], sink_tokens=16, seed=12)
    cuts = [4, 2, 3]
    got = _decode(w, terms=2, num_splits=4, row_splits=torch.tensor(cuts, dtype=torch.int32, device="cuda"))
    for row, parts in enumerate(cuts):
        uniform = _decode(w, terms=2, num_splits=parts)
        assert torch.equal(got[row], uniform[row]), (row, parts)
        want, _, _ = _oracle_decode(w, terms=2, scale_mode="amax6", rotate=False, num_splits=parts, bf16_split=True)
        _check(got[row], want[row], f"row {row} in {parts} parts")
    with pytest.raises(ValueError):
        _decode(w, terms=2, num_splits=4, row_splits=torch.tensor(cuts, dtype=torch.int64, device="cuda"))


def test_decode_row_order_changes_nothing():
    """A launch order (longest rows first) never changes the result; a non-permutation is refused
    unless the metadata is trusted."""
    from bdfp4.workload import build_workload

    lengths = [200, 3000, 129, 1500, 64, 2600, 900]
    w = build_workload(rows=len(lengths), heads_q=8, heads_kv=2, seq_lens=lengths, sink_tokens=16, seed=23)
    want = _decode(w, terms=2)
    order = torch.argsort(w.seqused_fp4, descending=True).to(torch.int32)
    assert torch.equal(_decode(w, terms=2, row_order=order), want)
    assert torch.equal(_decode(w, terms=2, num_splits=3, row_order=order), _decode(w, terms=2, num_splits=3))
    with pytest.raises(ValueError):
        _decode(w, terms=2, row_order=torch.zeros_like(order))
    with pytest.raises(ValueError):
        _decode(w, terms=2, row_order=order[:-1].contiguous())


def test_decode_caller_buffers_and_error_word():
    """Caller-owned output and scratch; nothing else is written."""
    from bdfp4.workload import build_workload
    from nvfp4_decode_kernel import split_partial_count

    w = build_workload(rows=3, heads_q=8, heads_kv=2, seq_lens=[400, 900, 131], sink_tokens=16, seed=12)
    rows, hq = 3, 8
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    parts = split_partial_count(rows, 2, 4, residual=True, sms=sms)
    out = torch.full((rows + 2, hq, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    scratch = dict(
        query_padded_scratch=torch.zeros(rows + 1, 128, hq, 128, dtype=torch.bfloat16, device="cuda"),
        query_fp4_scratch=torch.full((rows + 1, 1, hq, 64), 255, dtype=torch.uint8, device="cuda"),
        query_scales_scratch=torch.zeros(rows + 1, 1, hq, 2, 32, 4, 4, dtype=torch.uint8, device="cuda"),
        split_partial_scratch=torch.full((parts * rows * hq * 128,), float("nan"), device="cuda"),
        split_lse_scratch=torch.full((parts * rows * hq,), float("nan"), device="cuda"),
    )
    got = _decode(w, terms=1, num_splits=4, out=out, trusted_metadata=True, **scratch)
    assert got.data_ptr() == out.data_ptr() and got.shape[0] == rows
    assert bool((out[rows:] == 7.0).all())
    want, _, _ = _oracle_decode(w, terms=1, scale_mode="amax6", rotate=False, num_splits=4, bf16_split=True)
    _check(got, want, "caller buffers")


def test_plain_attention_distance_reported():
    """Distance to the plain dequantise-then-attend result (BF16 query, exact softmax): reported,
    and bounded loosely, because the FP4 probability operand alone costs about 9e-2 mean-rel."""
    from bdfp4.workload import build_workload

    w = build_workload(rows=1, heads_q=8, heads_kv=2, seq_lens=[2048], sink_tokens=16, seed=21, keep_source=True)
    out = _decode(w, terms=2).float().cpu()
    kc, ks, vc, vs = _cpu_cache(w)
    ids = w.page_table[0, :15].cpu().long()
    q = w.query[0].cpu().float()
    k_src, v_src = (t.cpu().float() for t in w.kept[0])
    errs = []
    for h in range(2):
        k = oracle.dequantize_key_pages(kc[ids][:, :, h:h + 1], ks[ids][:, h:h + 1]).reshape(-1, 128)
        v = oracle.dequantize_value_pages(vc[ids][:, h:h + 1], vs[ids][:, h:h + 1]).reshape(-1, 128)
        k[:16], v[:16] = k_src[:16, h], v_src[:16, h]
        k = torch.cat([k, k_src[1920:, h]])
        v = torch.cat([v, v_src[1920:, h]])
        want = oracle.plain_attention(q[4 * h:4 * h + 4], k, v, 128 ** -0.5)
        errs.append(((out[0, 4 * h:4 * h + 4] - want).abs().mean() / want.abs().mean()).item())
    print(f"mean-rel distance to plain dequantise-then-attend: {max(errs):.3e}")
    assert max(errs) < 0.3


def test_decode_is_cuda_graph_capturable():
    """With caller-owned scratch the whole call (query quantizer, decode, split merge) allocates
    and synchronises nothing, so it captures into a CUDA graph; a replay follows changed inputs."""
    from bdfp4.workload import build_workload
    from nvfp4_decode_kernel import DecodeTailWrite, fp4_decode, split_partial_count

    rows, hq, hkv = 4, 8, 2
    w = build_workload(rows=rows, heads_q=hq, heads_kv=hkv, seq_lens=[700, 129, 2048, 400], sink_tokens=16, seed=31,
                       key_scale_mode="four_six", rotate=True, page_tokens=64)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    parts = split_partial_count(rows, hkv, 3, residual=True, sms=sms)
    scratch = dict(
        query_padded_scratch=torch.zeros(rows, 128, hq, 128, dtype=torch.bfloat16, device="cuda"),
        query_fp4_scratch=torch.zeros(rows, 1, hq, 64, dtype=torch.uint8, device="cuda"),
        query_scales_scratch=torch.zeros(rows, 1, hq, 2, 32, 4, 4, dtype=torch.uint8, device="cuda"),
        query_fp4_second_scratch=torch.zeros(rows, 1, hq, 64, dtype=torch.uint8, device="cuda"),
        query_scales_second_scratch=torch.zeros(rows, 1, hq, 2, 32, 4, 4, dtype=torch.uint8, device="cuda"),
        split_partial_scratch=torch.empty(parts * rows * hq * 128, device="cuda"),
        split_lse_scratch=torch.empty(parts * rows * hq, device="cuda"),
        split_merge_counters=torch.zeros(rows * hkv, dtype=torch.int32, device="cuda"),
    )
    query = w.query.clone()
    new_key = torch.zeros(rows, hkv, 128, dtype=torch.bfloat16, device="cuda")
    new_value = torch.zeros_like(new_key)
    seq_lens = torch.tensor(w.seq_lens, dtype=torch.int32, device="cuda")
    out = torch.empty(rows, hq, 128, dtype=torch.bfloat16, device="cuda")

    def step():
        tail = DecodeTailWrite(new_key, new_value, w.tail_key[0], w.tail_value[0], w.slot_ids, seq_lens, w.seqused_fp4,
                               True, None, 16)
        return fp4_decode(
            query, *w.regions, w.page_table, w.seqused_fp4, residual_key_pages_bf16=w.tail_key[0],
            residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids,
            seqused_residual=w.seqused_residual, seqused_sink=w.seqused_sink, out=out, trusted_metadata=True,
            num_splits=3, query_terms=2, query_rotation="hadamard", tail_write=tail, **scratch)

    gen = torch.Generator(device="cuda").manual_seed(1)

    def fresh_inputs():
        query.copy_(torch.randn(rows, hq, 128, generator=gen, device="cuda").to(torch.bfloat16))
        new_key.copy_(torch.randn(rows, hkv, 128, generator=gen, device="cuda").to(torch.bfloat16))
        new_value.copy_(torch.randn(rows, hkv, 128, generator=gen, device="cuda").to(torch.bfloat16))

    fresh_inputs()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()  # warm-up outside capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(2):
        fresh_inputs()
        graph.replay()
        replayed = out.clone()
        eager = step().clone()
        assert torch.equal(replayed, eager)
    assert torch.cuda.memory_allocated() - before < (1 << 20)  # the capture held no sizeable allocation


@pytest.mark.parametrize("p_mode,tau", [("amax6", None), ("amax2_or_amax6", None), ("amax2_or_amax6_c8", 2.0),
                                        ("amax2_or_amax6", 0.3)])
def test_decode_probability_scale_modes(p_mode, tau, monkeypatch):
    """Every probability-scale rule the kernel has, and a threshold away from the default, on the
    grouped-query kernel (the rule and tau are launch arguments read from the environment)."""
    from bdfp4.workload import build_workload

    monkeypatch.setenv("NVFP4_P_SCALE_MODE", p_mode)
    if tau is not None:
        monkeypatch.setenv("NVFP4_P_SCALE_TAU", str(tau))
    w = build_workload(rows=3, heads_q=8, heads_kv=2, seq_lens=[900, 1700, 140], sink_tokens=16, seed=41)
    out = _decode(w, terms=2)
    want, _, _ = _oracle_decode(w, terms=2, scale_mode="amax6", rotate=False, p_mode=p_mode,
                                tau=oracle.DEFAULT_P_TAU if tau is None else tau)
    _check(out, want, f"{p_mode} tau={tau}")
    if tau is not None:
        # The threshold is live: the default one gives a different answer on the same inputs. (With
        # N(0,1) scores a group of sixteen almost always holds a probability above the default 21/1024
        # of the row maximum, so the thresholds tried here are large enough to move most groups to the
        # amax/2 scale.)
        monkeypatch.delenv("NVFP4_P_SCALE_TAU")
        assert not torch.equal(_decode(w, terms=2), out)


@pytest.mark.parametrize("heads_q,heads_kv", [(16, 2), (32, 2)])
@pytest.mark.parametrize("num_splits,fused", [(1, False), (2, False), (5, True)])
def test_decode_wide_groups_with_tail_sink_and_splits(heads_q, heads_kv, num_splits, fused):
    """Eight and sixteen query heads per KV head over the BF16 tail, the sink, split-KV and the
    fused merge (the paths the four-head cases above cover for G = 4)."""
    from bdfp4.workload import build_workload

    lengths = [1300, 129, 700, 2048, 90]
    w = build_workload(rows=len(lengths), heads_q=heads_q, heads_kv=heads_kv, seq_lens=lengths, sink_tokens=16,
                       seed=heads_q + num_splits, key_scale_mode="four_six", rotate=True)
    extra = {}
    if fused:
        extra = dict(split_merge_counters=torch.zeros(len(lengths) * heads_kv, dtype=torch.int32, device="cuda"))
    out = _decode(w, terms=2, scale_mode="four_six", rotate=True, num_splits=num_splits, **extra)
    want, _, _ = _oracle_decode(w, terms=2, scale_mode="four_six", rotate=True, num_splits=num_splits,
                                bf16_split=num_splits > 1)
    _check(out, want, f"G={heads_q // heads_kv} splits={num_splits}")


@pytest.mark.parametrize("heads_q,heads_kv,page_tokens", [(8, 2, 128), (16, 2, 128), (16, 2, 64), (32, 2, 128)])
def test_decode_rescales_when_the_maximum_moves_late(heads_q, heads_kv, page_tokens):
    """The oldest tokens (reached last) score far above everything before them, so the running
    maximum moves by more than the stale-maximum rule tolerates near the end of the walk and the
    sums accumulated so far are rescaled; with eight or more rows per thread the per-row statistics
    involved live in shared memory."""
    from bdfp4.workload import build_workload

    w = build_workload(rows=3, heads_q=heads_q, heads_kv=heads_kv, seq_lens=[1500, 700, 2300], sink_tokens=16,
                       seed=53, loud_prefix=200, page_tokens=page_tokens)
    out = _decode(w, terms=2)
    kwargs = dict(terms=2, scale_mode="amax6", rotate=False)
    if page_tokens == 64:
        from tests.test_gpu_page64 import _oracle_decode as oracle64

        want = oracle64(w, terms=2, rotate=False)
    else:
        want, _, _ = _oracle_decode(w, **kwargs)
    _check(out, want, f"late maximum, G={heads_q // heads_kv}, {page_tokens}-token pages", large_outputs=True)
    # the scenario is the intended one: without the loud prefix the same rows give another answer,
    # and the oracle with the stale-maximum rule switched off (always move) differs from the gate's
    quiet = build_workload(rows=3, heads_q=heads_q, heads_kv=heads_kv, seq_lens=[1500, 700, 2300], sink_tokens=16,
                           seed=53, page_tokens=page_tokens)
    assert not torch.equal(_decode(quiet, terms=2), out)


def test_decode_with_tensor_scales():
    """FP32 per-tensor scales on K, V and Q (no reference counterpart, so this parity is unpinned:
    the oracle restates the CUDA path's own definition). 1.0 must leave every byte as it was."""
    from bdfp4.workload import build_workload

    common = dict(rows=2, heads_q=8, heads_kv=2, seq_lens=[1100, 400], sink_tokens=16, seed=61,
                  key_scale_mode="four_six", rotate=True)
    plain = build_workload(**common)
    ones = build_workload(key_tensor_scale=1.0, value_tensor_scale=1.0, **common)
    assert torch.equal(plain.blocks, ones.blocks)
    w = build_workload(key_tensor_scale=3.0, value_tensor_scale=0.37, **common)
    assert not torch.equal(plain.blocks, w.blocks)
    kc, ks, vc, vs = _cpu_cache(w)
    want_plain = _cpu_cache(plain)
    assert not torch.equal(ks, want_plain[1]) and not torch.equal(vs, want_plain[3])
    out = _decode(w, terms=2, scale_mode="four_six", rotate=True, tensor_scales=(3.0, 1.7, 0.37))
    want, _, _ = _oracle_decode(w, terms=2, scale_mode="four_six", rotate=True, query_scale=1.7)
    _check(out, want, "tensor scales")
    # the scales cancel: the result is close to the unscaled cache's (not equal: other block scales)
    base = _decode(plain, terms=2, scale_mode="four_six", rotate=True).float()
    assert float((out.float() - base).abs().mean() / base.abs().mean()) < 0.3
