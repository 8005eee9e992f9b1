"""Bit-exact parity of the CUDA quantizers (through the C ABI) with the CPU oracle."""

import pytest
import torch

from oracle import nvfp4_oracle as oracle

pytestmark = pytest.mark.gpu

MODES = ["amax6", "four_six", "four_six_sixhalf"]


def _inputs(pages, heads, seed, outliers=True):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(pages, 128, heads, 128, generator=gen)
    if outliers:
        for h in range(heads):
            ch = torch.randperm(128, generator=gen)[:4]
            x[:, :, h, ch] *= torch.exp(1.5 * torch.randn(4, generator=gen))
    return x.to(torch.bfloat16)


def _adversarial_page(heads):
    """One page whose token rows are the golden generator's adversarial rows, tiled."""
    import numpy as np
    from pathlib import Path

    golden = np.load(Path(__file__).parent / "golden" / "reference_vectors.npz")
    rows = torch.from_numpy(golden["quant_x"])  # [49, 128]
    page = rows.repeat(3, 1)[:128]  # [128,128]
    return page[None, :, None, :].repeat(1, 1, heads, 1).to(torch.bfloat16)


def _scale_bytes(view, pages, heads):
    """The strided scale view -> [pages, H, 1024] bytes on the CPU."""
    flat = torch.empty(pages, heads, 1024, dtype=torch.uint8)
    v = view.view(torch.uint8).cpu()  # (pages,32,4,1,4,2,H)
    off = oracle.scale_tile_offsets()  # [128,8]
    r = torch.arange(128)
    for g in range(8):
        flat[:, :, off[:, g]] = v[:, r % 32, r // 32, 0, g % 4, g // 4, :].permute(0, 2, 1)
    return flat


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("heads", [1, 2, 8])
def test_key_pages(mode, heads):
    from nvfp4_decode_kernel.quantize_kv_kernel import quantize_key_pages

    x = torch.cat([_inputs(3, heads, 11 + heads), _adversarial_page(heads)])
    codes, scales = quantize_key_pages(x.cuda(), mode)
    want_codes, want_scales = oracle.quantize_key_pages(x, mode)
    assert torch.equal(codes.cpu(), want_codes)
    assert torch.equal(_scale_bytes(scales, x.shape[0], heads), want_scales)


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("heads", [1, 2, 8])
def test_value_pages(mode, heads):
    from nvfp4_decode_kernel.quantize_kv_kernel import quantize_value_pages

    x = torch.cat([_inputs(3, heads, 23 + heads, outliers=False), _adversarial_page(heads)])
    codes, scales = quantize_value_pages(x.cuda(), mode)
    want_codes, want_scales = oracle.quantize_value_pages(x, mode)
    assert torch.equal(codes.cpu(), want_codes)
    assert torch.equal(_scale_bytes(scales, x.shape[0], heads), want_scales)


@pytest.mark.parametrize("rotate,shift_dtype", [(True, None), (False, torch.float32), (True, torch.float32),
                                                (True, torch.bfloat16)])
def test_key_cache_basis(rotate, shift_dtype):
    """Hadamard rotation and key shift on the way into the pages (scatter through a work table)."""
    from nvfp4_decode_kernel.quantize_kv_kernel import KVCacheWriter, _allocate_scales

    heads, pages = 2, 4
    x = _inputs(pages, heads, 5)
    gen = torch.Generator().manual_seed(9)
    shift = None
    if shift_dtype is not None:
        shift = (0.3 * torch.randn(3, heads, 128, generator=gen)).to(shift_dtype)
    layer = 1
    codes = torch.zeros(pages + 2, 128, heads, 64, dtype=torch.uint8, device="cuda")
    _, scales = _allocate_scales(pages + 2, heads, 1, 2, "cuda")
    scales.view(torch.uint8).zero_()
    regions = (codes, scales, None, None)
    writer = KVCacheWriter(regions=regions, key_scale_mode="four_six", rotate_key=rotate,
                           key_shift=None if shift is None else shift.cuda())
    dest = torch.tensor([4, -1, 0, 5], dtype=torch.int32, device="cuda")
    src = torch.tensor([0, 128, 256, 384], dtype=torch.int32, device="cuda")
    writer(x.reshape(-1, heads, 128).cuda(), None, regions, src, dest, layer=layer)
    want_codes, want_scales = oracle.quantize_key_pages(
        x, "four_six", rotate=rotate, shift=None if shift is None else shift[layer].float())
    got_scales = _scale_bytes(scales, pages + 2, heads)
    for w, d in enumerate([4, -1, 0, 5]):
        if d < 0:
            continue
        assert torch.equal(codes[d].cpu(), want_codes[w])
        assert torch.equal(got_scales[d], want_scales[w])
    for untouched in (1, 2, 3):
        assert int(codes[untouched].sum()) == 0


def test_per_layer_seal():
    """The per-layer form: one launch quantizes the same work items of every layer through a
    [4, layers] base-address table."""
    from nvfp4_decode_kernel.quantize_kv_kernel import KVCacheWriter, _allocate_scales

    heads, layers, pages = 2, 3, 2
    k = _inputs(layers * pages, heads, 31).reshape(layers, pages * 128, heads, 128)
    v = _inputs(layers * pages, heads, 32, outliers=False).reshape(layers, pages * 128, heads, 128)
    kc = [torch.zeros(4, 128, heads, 64, dtype=torch.uint8, device="cuda") for _ in range(layers)]
    vc = [torch.zeros(4, heads, 128, 64, dtype=torch.uint8, device="cuda") for _ in range(layers)]
    ks = [_allocate_scales(4, heads, 1, 2, "cuda")[1] for _ in range(layers)]
    vs = [_allocate_scales(4, heads, 1, 2, "cuda")[1] for _ in range(layers)]
    bases = torch.tensor([[t.data_ptr() for t in group] for group in (kc, ks, vc, vs)], dtype=torch.int64,
                         device="cuda")
    regions = (kc[0], ks[0], vc[0], vs[0])
    writer = KVCacheWriter(regions=regions, key_scale_mode="four_six", value_scale_mode="amax6",
                           destination_bases=bases)
    src = torch.tensor([0, 128], dtype=torch.int32, device="cuda")
    dest = torch.tensor([3, 1], dtype=torch.int32, device="cuda")
    writer(k.reshape(-1, heads, 128).cuda(), v.reshape(-1, heads, 128).cuda(), regions, src, dest)
    for layer in range(layers):
        want_kc, want_ks = oracle.quantize_key_pages(k[layer].reshape(pages, 128, heads, 128), "four_six")
        want_vc, want_vs = oracle.quantize_value_pages(v[layer].reshape(pages, 128, heads, 128), "amax6")
        got_ks, got_vs = _scale_bytes(ks[layer], 4, heads), _scale_bytes(vs[layer], 4, heads)
        for w, d in enumerate([3, 1]):
            assert torch.equal(kc[layer][d].cpu(), want_kc[w])
            assert torch.equal(vc[layer][d].cpu(), want_vc[w])
            assert torch.equal(got_ks[d], want_ks[w])
            assert torch.equal(got_vs[d], want_vs[w])


@pytest.mark.parametrize("terms", [1, 2])
@pytest.mark.parametrize("rotate", [False, True])
@pytest.mark.parametrize("heads_q,heads_kv", [(8, 2), (32, 8), (32, 4), (5, 5)])
def test_query(terms, rotate, heads_q, heads_kv):
    from nvfp4_decode_kernel._quantize import quantize_query

    rows = 5
    gen = torch.Generator().manual_seed(heads_q * 7 + terms)
    q = torch.randn(rows + 2, heads_q, 128, generator=gen).to(torch.bfloat16)
    idx = torch.tensor([6, 0, 3, 3, 1], dtype=torch.int32)
    padded = torch.zeros(rows, 128, heads_q, 128, dtype=torch.bfloat16, device="cuda")
    got = quantize_query(q.cuda(), row_indices=idx.cuda(), query_padded_out=padded, heads_kv=heads_kv,
                         query_terms=terms, scale_mode="four_six", rotation="hadamard" if rotate else "none")
    want = oracle.quantize_query(q[idx.long()], heads_kv, scale_mode="four_six", terms=terms, rotate=rotate)
    for term in range(terms):
        codes = got[2 * term].view(torch.uint8).cpu()
        assert torch.equal(codes, want["codes"][term])
        storage = got[2 * term + 1]
        raw = torch.as_strided(storage, (rows, heads_q * 1024), (heads_q * 1024, 1)).cpu()
        assert torch.equal(raw.reshape(rows, 1, heads_q, 2, 32, 4, 4), want["scales"][term])
    assert torch.equal(padded[:, 0].cpu(), want["padded"])
    assert int(padded[:, 1:].abs().sum()) == 0


def test_combine():
    import bdfp4

    gen = torch.Generator().manual_seed(3)
    parts, rows, heads = 5, 3, 8
    po = torch.randn(parts, rows, heads, 128, generator=gen)
    lse = torch.randn(parts, rows, heads, generator=gen) * 3
    lse[1] = -torch.inf
    po[1] = float("nan")
    lse[:, 2, 3] = -torch.inf  # every part empty
    out = torch.empty(rows, heads, 128, dtype=torch.bfloat16, device="cuda")
    bdfp4.combine(po.cuda(), lse.cuda(), parts, rows, heads, out, out.stride(0), bdfp4.current_stream(out.device))
    want = oracle.combine_partials(po, lse)
    torch.testing.assert_close(out.cpu().float(), want.float(), rtol=1e-2, atol=1e-3)
    assert float(out[2, 3].abs().sum()) == 0.0
