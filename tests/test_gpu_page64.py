"""64-token cache pages: the CUDA quantizers and the decode kernel against the CPU oracle.

The reference serves 128-token pages only, so no bytes of the reference pin this layout. The
gates are the same as for 128-token pages: codes and scale bytes bit-exact against the oracle's
statement of the layout, whose values are those of the 128-token page holding the same tokens
(checked on the CPU in test_oracle_page64.py); attention within max |err| <= 1e-2 and mean
relative error <= 1e-3 of the oracle, and equal to the 128-token-page result on the same tokens.
"""

import pytest
import torch

from oracle import nvfp4_oracle as oracle

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_REL = 1e-2, 1e-3
MODES = ["amax6", "four_six", "four_six_sixhalf"]


def _inputs(pages, heads, seed, outliers=True):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(pages, 64, heads, 128, generator=gen)
    if outliers:
        for h in range(heads):
            ch = torch.randperm(128, generator=gen)[:4]
            x[:, :, h, ch] *= torch.exp(1.5 * torch.randn(4, generator=gen))
    return x.to(torch.bfloat16)


def _flat(view, heads, nbytes=512):
    """A strided scale view -> [pages, H, nbytes] bytes on the CPU."""
    u8 = view.view(torch.uint8)
    return u8.as_strided((u8.shape[0], heads, nbytes), (u8.stride(0), nbytes, 1), u8.storage_offset()).cpu()


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("heads", [1, 2, 8])
def test_key_pages(mode, heads):
    from nvfp4_decode_kernel.quantize_kv_kernel import quantize_key_pages

    x = _inputs(5, heads, 41 + heads)
    codes, scales = quantize_key_pages(x.cuda(), mode)
    assert tuple(codes.shape) == (5, 64, heads, 64)
    want_codes, want_scales = oracle.quantize_key_pages(x, mode)
    assert torch.equal(codes.cpu(), want_codes)
    assert torch.equal(_flat(scales, heads), want_scales)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("heads", [1, 2, 8])
def test_value_pages(mode, heads):
    from nvfp4_decode_kernel.quantize_kv_kernel import quantize_value_pages

    x = _inputs(5, heads, 57 + heads, outliers=False)
    codes, scales = quantize_value_pages(x.cuda(), mode)
    assert tuple(codes.shape) == (5, heads, 128, 32)
    want_codes, want_scales = oracle.quantize_value_pages(x, mode)
    assert torch.equal(codes.cpu(), want_codes)
    assert torch.equal(_flat(scales, heads), want_scales)


def _cpu_cache(w):
    blocks, h = w.blocks.cpu(), w.heads_kv
    key_codes = blocks[:, :4096 * h].reshape(-1, h, 64, 64).permute(0, 2, 1, 3)
    key_scales = blocks[:, 4096 * h:4608 * h].reshape(-1, h, 512)
    value_codes = blocks[:, 4608 * h:8704 * h].reshape(-1, h, 128, 32)
    value_scales = blocks[:, 8704 * h:9216 * h].reshape(-1, h, 512)
    return key_codes, key_scales, value_codes, value_scales


def test_writer_scatter_rotation_and_shift():
    """The paged writer (work table, Hadamard rotation, key shift) fills 64-token pages with the
    oracle's bytes."""
    from bdfp4.workload import build_workload

    w = build_workload(rows=2, heads_q=8, heads_kv=2, seq_lens=[700, 390], sink_tokens=16, seed=3,
                       key_scale_mode="four_six", rotate=True, key_shift=True, keep_source=True, page_tokens=64)
    kc, ks, vc, vs = _cpu_cache(w)
    for row, n in enumerate(w.seq_lens):
        fp4 = int(w.seqused_fp4[row])
        ids = w.page_table[row, :fp4 // 64].cpu().long()
        k_src, v_src = (t.cpu()[:fp4].reshape(-1, 64, 2, 128) for t in w.kept[row])
        want_kc, want_ks = oracle.quantize_key_pages(k_src, "four_six", rotate=True, shift=w.key_shift[0].cpu())
        want_vc, want_vs = oracle.quantize_value_pages(v_src, "amax6")
        assert torch.equal(kc[ids], want_kc) and torch.equal(ks[ids], want_ks)
        assert torch.equal(vc[ids], want_vc) and torch.equal(vs[ids], want_vs)


def _decode(w, *, terms, rotate, num_splits=1):
    from nvfp4_decode_kernel import fp4_decode

    return fp4_decode(
        w.query, *w.regions, w.page_table, w.seqused_fp4, residual_key_pages_bf16=w.tail_key[0],
        residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids,
        seqused_residual=w.seqused_residual, seqused_sink=w.seqused_sink, query_terms=terms, scale_mode="amax6",
        query_rotation="hadamard" if rotate else "none", num_splits=num_splits)


def _oracle_decode(w, *, terms, rotate, num_splits=1):
    kc, ks, vc, vs = _cpu_cache(w)
    q = oracle.quantize_query(w.query.cpu(), w.heads_kv, scale_mode="amax6", terms=terms, rotate=rotate)
    return oracle.decode_reference(
        query_values=q["values"], query_padded=q["padded"], key_codes=kc, key_scales=ks, value_codes=vc,
        value_scales=vs, page_table=w.page_table.cpu(), seqused_fp4=w.seqused_fp4.cpu(), heads_kv=w.heads_kv,
        softmax_scale=128 ** -0.5, num_splits=num_splits, bf16_split=num_splits > 1,
        tail_key=w.tail_key[0].cpu(), tail_value=w.tail_value[0].cpu(), tail_slot_ids=w.slot_ids.cpu(),
        seqused_residual=w.seqused_residual.cpu(), seqused_sink=w.seqused_sink.cpu())[0]


def _check(got, want, label):
    got, want = got.float().cpu(), want.float()
    assert torch.isfinite(got).all(), label
    err = (got - want).abs()
    mean_rel = float(err.mean() / want.abs().mean().clamp_min(1e-12))
    assert float(err.max()) <= MAX_ABS, f"{label} max abs err {float(err.max()):.3e}"
    assert mean_rel <= MEAN_REL, f"{label} mean rel err {mean_rel:.3e}"


@pytest.mark.parametrize("heads_q,heads_kv,terms,rotate", [(8, 2, 2, True), (8, 1, 1, False), (16, 1, 2, True)])
def test_decode_matches_oracle_and_128_token_pages(heads_q, heads_kv, terms, rotate):
    from bdfp4.workload import build_workload

    lengths = [1500, 129, 128, 77, 2048, 641]
    common = dict(rows=len(lengths), heads_q=heads_q, heads_kv=heads_kv, seq_lens=lengths, sink_tokens=16, seed=5,
                  key_scale_mode="four_six", rotate=rotate)
    w64 = build_workload(page_tokens=64, **common)
    out64 = _decode(w64, terms=terms, rotate=rotate)
    _check(out64, _oracle_decode(w64, terms=terms, rotate=rotate), "64-token pages")
    # same seed, same tokens: only the physical placement differs
    w128 = build_workload(page_tokens=128, **common)
    from nvfp4_decode_kernel import fp4_decode

    out128 = fp4_decode(
        w128.query, *w128.regions, w128.page_table, w128.seqused_fp4, residual_key_pages_bf16=w128.tail_key[0],
        residual_value_pages_bf16=w128.tail_value[0], residual_page_ids=w128.slot_ids,
        seqused_residual=w128.seqused_residual, seqused_sink=w128.seqused_sink, query_terms=terms,
        scale_mode="amax6", query_rotation="hadamard" if rotate else "none")
    assert torch.equal(w64.query, w128.query)
    _check(out64, out128.float().cpu(), "64- vs 128-token pages")


@pytest.mark.parametrize("num_splits", [2, 5])
def test_decode_split_kv(num_splits):
    from bdfp4.workload import build_workload

    w = build_workload(rows=3, heads_q=8, heads_kv=2, seq_lens=[1800, 260, 1031], sink_tokens=16, seed=8,
                       page_tokens=64)
    out = _decode(w, terms=2, rotate=False, num_splits=num_splits)
    _check(out, _oracle_decode(w, terms=2, rotate=False, num_splits=num_splits), f"splits={num_splits}")


def test_odd_page_table_width_and_bad_page_report():
    """A table with an odd number of columns serves whole 128-token steps only; an entry outside
    the cache is clamped and reported in the error word."""
    import bdfp4
    from bdfp4.workload import build_workload

    w = build_workload(rows=1, heads_q=4, heads_kv=1, seq_lens=[600], sink_tokens=16, seed=9, page_tokens=64)
    table = torch.cat([w.page_table, torch.zeros(1, 1, dtype=torch.int32, device="cuda")], dim=1).contiguous()
    assert table.shape[1] % 2 == 1
    w.page_table = table
    out = _decode(w, terms=1, rotate=False)
    _check(out, _oracle_decode(w, terms=1, rotate=False), "odd table width")
