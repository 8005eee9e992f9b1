"""The MXFP4 arm (E2M1 codes, one E8M0 power-of-two scale per 32 values) on the GPU.

Quantizers: codes and scale bytes bit-exact against ``oracle/mxfp4_oracle.py``, which is pinned to
the reference's own ``mxfp4_quantize`` (three exponent rules) by ``tests/test_oracle_mxfp4.py``.
Attention: max |err| <= 1e-2 and mean relative error <= 1e-3 in BF16 against the oracle's
composition of those pieces with the reference's MXFP4 probability operand
(``mxfp4_probability_quantize``). The reference has no CPU model of whole MXFP4 attention, so that
composition is this repository's: parity of the attention gate is unpinned, the pieces are pinned.
"""

import pytest
import torch

from oracle import mxfp4_oracle as mx
from oracle import tile_check

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_REL = 1e-2, 1e-3
RULES = ["ocp", "round_up", "search"]


def _pages(pages, heads, seed, outliers=True):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(pages, 128, heads, 128, generator=gen)
    if outliers:
        for h in range(heads):
            ch = torch.randperm(128, generator=gen)[:4]
            x[:, :, h, ch] *= torch.exp(1.5 * torch.randn(4, generator=gen))
    x[0, :3] = 0.0           # all-zero groups: exponent -127, byte 0
    x[1, 5, 0, :32] = 6.0    # a maximum exactly on the E2M1 top under the OCP scale
    x[1, 6, 0, :32] = 6.0001
    return x.to(torch.bfloat16)


def _flat(view, heads, nbytes=512):
    u8 = view.view(torch.uint8)
    return u8.as_strided((u8.shape[0], heads, nbytes), (u8.stride(0), nbytes, 1), u8.storage_offset()).cpu()


@pytest.mark.parametrize("rule", RULES)
@pytest.mark.parametrize("heads", [1, 2, 8])
def test_key_pages(rule, heads):
    from nvfp4_decode_kernel.quantize_kv_kernel import quantize_key_pages

    x = _pages(4, heads, 11 + heads)
    codes, scales = quantize_key_pages(x.cuda(), f"mxfp4_{rule}")
    assert scales.dtype is torch.float8_e8m0fnu and tuple(codes.shape) == (4, 128, heads, 64)
    want_codes, want_scales = mx.quantize_key_pages(x, rule)
    assert torch.equal(codes.cpu(), want_codes)
    assert torch.equal(_flat(scales, heads), want_scales)


@pytest.mark.parametrize("rule", RULES)
@pytest.mark.parametrize("heads", [1, 2, 8])
def test_value_pages(rule, heads):
    from nvfp4_decode_kernel.quantize_kv_kernel import quantize_value_pages

    x = _pages(4, heads, 23 + heads, outliers=False)
    codes, scales = quantize_value_pages(x.cuda(), f"mxfp4_{rule}")
    assert tuple(codes.shape) == (4, heads, 128, 64)
    want_codes, want_scales = mx.quantize_value_pages(x, rule)
    assert torch.equal(codes.cpu(), want_codes)
    assert torch.equal(_flat(scales, heads), want_scales)


@pytest.mark.parametrize("rule", RULES)
@pytest.mark.parametrize("heads_q,heads_kv", [(8, 2), (4, 4), (32, 2)])
@pytest.mark.parametrize("terms,rotate", [(1, False), (2, True)])
def test_query(rule, heads_q, heads_kv, terms, rotate):
    from nvfp4_decode_kernel._quantize import quantize_query

    gen = torch.Generator().manual_seed(heads_q + terms)
    q = (torch.randn(5, heads_q, 128, generator=gen) * 2.0).to(torch.bfloat16)
    padded = torch.zeros(5, 128, heads_q, 128, dtype=torch.bfloat16, device="cuda")
    got = quantize_query(q.cuda(), query_padded_out=padded, heads_kv=heads_kv, query_terms=terms,
                         scale_mode=f"mxfp4_{rule}", rotation="hadamard" if rotate else "none")
    want = mx.quantize_query(q, heads_kv, rule=rule, terms=terms, rotate=rotate)
    assert torch.equal(padded[:, 0].cpu(), want["padded"])
    for term in range(terms):
        codes, scales = got[2 * term], got[2 * term + 1]
        assert torch.equal(codes.view(torch.uint8).cpu(), want["codes"][term])
        assert tuple(scales.shape) == (32, 4, 1, 4, 1, heads_kv, 5)
        storage = scales.as_strided((5, 1, heads_q, 1, 32, 4, 4), (heads_q * 512, heads_q * 512, 512, 512, 16, 4, 1))
        assert torch.equal(storage.cpu(), want["scales"][term])


def test_writer_scatter_rotation_shift_and_page_bound():
    """The paged writer under MXFP4 (work table, Hadamard, key shift) fills the oracle's bytes, and a
    destination past the cache is skipped and reported instead of written."""
    import bdfp4
    from bdfp4.workload import build_workload, carve_cache
    from nvfp4_decode_kernel.quantize_kv_kernel import KVCacheWriter

    w = build_workload(rows=2, heads_q=8, heads_kv=2, seq_lens=[700, 390], sink_tokens=16, seed=3,
                       key_scale_mode="mxfp4_search", value_scale_mode="mxfp4_ocp", rotate=True, key_shift=True,
                       keep_source=True)
    assert w.scale_format == "mxfp4"
    blocks = w.blocks.cpu()
    h = 2
    kc = blocks[:, :8192 * h].reshape(-1, 128, h, 64)
    ks = blocks[:, 8192 * h:8192 * h + 512 * h].reshape(-1, h, 512)
    vc = blocks[:, 9216 * h:17408 * h].reshape(-1, h, 128, 64)
    vs = blocks[:, 17408 * h:17408 * h + 512 * h].reshape(-1, h, 512)
    for row in range(2):
        fp4 = int(w.seqused_fp4[row])
        ids = w.page_table[row, :fp4 // 128].cpu().long()
        k_src, v_src = (t.cpu()[:fp4].reshape(-1, 128, 2, 128) for t in w.kept[row])
        want_kc, want_ks = mx.quantize_key_pages(k_src, "search", rotate=True, shift=w.key_shift[0].cpu())
        want_vc, want_vs = mx.quantize_value_pages(v_src, "ocp")
        assert torch.equal(kc[ids], want_kc) and torch.equal(ks[ids], want_ks)
        assert torch.equal(vc[ids], want_vc) and torch.equal(vs[ids], want_vs)
    # the unused second half of each scale region stays untouched (zero)
    assert int(blocks[:, 8192 * h + 512 * h:9216 * h].abs().sum()) == 0


def _decode(w, *, terms, rotate, rule="ocp", num_splits=1, **extra):
    from nvfp4_decode_kernel import fp4_decode

    return fp4_decode(
        w.query, *w.regions, w.page_table, w.seqused_fp4, residual_key_pages_bf16=w.tail_key[0],
        residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids,
        seqused_residual=w.seqused_residual, seqused_sink=w.seqused_sink, query_terms=terms,
        scale_mode=f"mxfp4_{rule}", query_rotation="hadamard" if rotate else "none", num_splits=num_splits, **extra)


def _check_all_tiles(w, out, label, **options):
    tiles = [(row, head) for row in range(w.rows) for head in range(w.heads_kv)]
    result = tile_check.check_tiles(w, out, tiles, **options)
    assert result["max_abs"] <= MAX_ABS, (label, result)
    assert result["mean_rel"] <= MEAN_REL, (label, result)


@pytest.mark.parametrize("heads_q,heads_kv,terms,rotate", [(8, 2, 1, False), (8, 2, 2, True), (16, 2, 2, True),
                                                           (32, 2, 1, False)])
def test_decode_matches_the_oracle(heads_q, heads_kv, terms, rotate):
    from bdfp4.workload import build_workload

    lengths = [1500, 129, 128, 77, 2048, 641]
    w = build_workload(rows=len(lengths), heads_q=heads_q, heads_kv=heads_kv, seq_lens=lengths, sink_tokens=16,
                       seed=7, key_scale_mode="mxfp4_search", value_scale_mode="mxfp4_ocp", rotate=rotate)
    out = _decode(w, terms=terms, rotate=rotate)
    _check_all_tiles(w, out, f"mxfp4 G={heads_q // heads_kv} terms={terms}", terms=terms, scale_mode="mxfp4_ocp",
                     rotate=rotate)


@pytest.mark.parametrize("num_splits", [2, 5])
def test_decode_split_kv(num_splits):
    from bdfp4.workload import build_workload

    w = build_workload(rows=3, heads_q=8, heads_kv=2, seq_lens=[1800, 260, 1031], sink_tokens=16, seed=8,
                       key_scale_mode="mxfp4_round_up", value_scale_mode="mxfp4_round_up")
    out = _decode(w, terms=2, rotate=False, rule="round_up", num_splits=num_splits)
    _check_all_tiles(w, out, f"mxfp4 splits={num_splits}", terms=2, scale_mode="mxfp4_round_up", rotate=False,
                     num_splits=num_splits, bf16_split=True)


def test_decode_late_maximum_and_refusals(monkeypatch):
    from bdfp4.workload import build_workload

    w = build_workload(rows=2, heads_q=8, heads_kv=2, seq_lens=[1500, 900], sink_tokens=16, seed=9,
                       key_scale_mode="mxfp4_ocp", value_scale_mode="mxfp4_ocp", loud_prefix=200)
    out = _decode(w, terms=1, rotate=False)
    _check_all_tiles(w, out, "mxfp4 late maximum", terms=1, scale_mode="mxfp4_ocp", rotate=False)
    # an NVFP4 query against an MXFP4 cache is a shape error, never a silent misread
    with pytest.raises(ValueError):
        from nvfp4_decode_kernel import fp4_decode

        fp4_decode(w.query, *w.regions, w.page_table, w.seqused_fp4)
    # the NVFP4 probability-scale overrides do not apply to MXFP4 and are refused, not ignored
    monkeypatch.setenv("NVFP4_P_SCALE_MODE", "amax6")
    with pytest.raises(ValueError):
        _decode(w, terms=1, rotate=False)
