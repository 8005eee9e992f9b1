"""The oracle's 64-token page layout carries the values of the reference's 128-token page.

The reference has no 64-token page; what pins the variant is that quantizing the same tokens as
two 64-token pages gives exactly the codes and scales of the one 128-token page (whose layout and
arithmetic are pinned by the reference's golden vectors), placed at the documented byte offsets.
"""

import torch

from oracle import nvfp4_oracle as oracle


def _pages(seed, heads=2, pages=3):
    gen = torch.Generator().manual_seed(seed)
    return torch.randn(pages, 128, heads, 128, generator=gen).to(torch.bfloat16)


def test_key_pages_hold_the_128_token_values():
    k = _pages(1)
    shift = 0.2 * torch.randn(2, 128, generator=torch.Generator().manual_seed(2))
    codes, scales = oracle.quantize_key_pages(k, "four_six", rotate=True, shift=shift)
    codes64, scales64 = oracle.quantize_key_pages(k.reshape(6, 64, 2, 128), "four_six", rotate=True, shift=shift)
    assert tuple(codes64.shape) == (6, 64, 2, 64) and tuple(scales64.shape) == (6, 2, 512)
    # code bytes: those of the 128-token page with each token's 16-byte chunks moved to j ^ ((t >> 1) & 3)
    plain = codes.reshape(6, 64, 2, 4, 16)
    for t in (0, 1, 2, 5, 63):
        for j in range(4):
            assert torch.equal(codes64.reshape(6, 64, 2, 4, 16)[:, t, :, j ^ ((t >> 1) & 3)], plain[:, t, :, j])
    # scale bytes: token t of the step, group g
    tile = scales.reshape(3, 2, 1024)
    for t in (0, 31, 32, 63, 64, 100, 127):
        for g in range(8):
            at128 = (g // 4) * 512 + (t % 32) * 16 + (t // 32) * 4 + g % 4
            half, u = divmod(t, 64)
            at64 = (g // 4) * 256 + (u % 32) * 8 + (u // 32) * 4 + g % 4
            assert torch.equal(scales64.reshape(3, 2, 2, 512)[:, half, :, at64], tile[:, :, at128])
    assert torch.equal(oracle.dequantize_key_pages(codes64, scales64).reshape(3, 128, 2, 128),
                       oracle.dequantize_key_pages(codes, scales))


def test_interleaving_two_key_scale_blocks_gives_the_mma_atoms():
    """What the decode kernel does in shared memory: rows of 8 bytes from the step's two pages,
    side by side, are the 16-byte rows of the 128-token tile's two atoms."""
    k = _pages(3, heads=1, pages=1)
    _, scales = oracle.quantize_key_pages(k, "amax6")
    _, scales64 = oracle.quantize_key_pages(k.reshape(2, 64, 1, 128), "amax6")
    first, second = scales64[0, 0].reshape(2, 32, 8), scales64[1, 0].reshape(2, 32, 8)
    merged = torch.cat([first, second], dim=-1).reshape(1024)
    assert torch.equal(merged, scales[0, 0])


def test_value_pages_hold_the_128_token_values():
    v = _pages(4)
    codes, scales = oracle.quantize_value_pages(v, "four_six")
    codes64, scales64 = oracle.quantize_value_pages(v.reshape(6, 64, 2, 128), "four_six")
    assert tuple(codes64.shape) == (6, 2, 128, 32) and tuple(scales64.shape) == (6, 2, 512)
    both = codes64.reshape(3, 2, 2, 128, 2, 16)
    plain = codes.reshape(3, 2, 128, 2, 2, 16)  # [.., channel, half page, chunk, 16]
    for c in (0, 3, 4, 7, 127):
        for j in range(2):
            for half in range(2):
                assert torch.equal(both[:, half, :, c, j ^ ((c >> 2) & 1)], plain[:, :, c, half, j])
    # a page's 512 scale bytes are one atom: the first (tokens 0-63) or second (64-127) of the tile
    tile = scales.reshape(3, 2, 2, 512)
    assert torch.equal(scales64.reshape(3, 2, 2, 512).permute(0, 2, 1, 3), tile)
    assert torch.equal(oracle.dequantize_value_pages(codes64, scales64).reshape(3, 128, 2, 128),
                       oracle.dequantize_value_pages(codes, scales))


def test_decode_reference_is_page_size_blind():
    gen = torch.Generator().manual_seed(7)
    k, v = _pages(11), _pages(12)
    q = torch.randn(1, 8, 128, generator=gen).to(torch.bfloat16)
    qq = oracle.quantize_query(q, 2, terms=2)
    common = dict(query_values=qq["values"], query_padded=qq["padded"], heads_kv=2, softmax_scale=128 ** -0.5,
                  seqused_fp4=torch.tensor([384]))
    kc, ks = oracle.quantize_key_pages(k)
    vc, vs = oracle.quantize_value_pages(v)
    want = oracle.decode_reference(key_codes=kc, key_scales=ks, value_codes=vc, value_scales=vs,
                                   page_table=torch.tensor([[2, 0, 1]]), **common)[0]
    order = torch.tensor([2, 0, 1])
    kc64, ks64 = oracle.quantize_key_pages(k[order].reshape(6, 64, 2, 128))
    vc64, vs64 = oracle.quantize_value_pages(v[order].reshape(6, 64, 2, 128))
    perm = torch.tensor([4, 1, 5, 0, 3, 2])  # physical home of the six 64-token pages
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(6)
    got = oracle.decode_reference(key_codes=kc64[inv], key_scales=ks64[inv], value_codes=vc64[inv],
                                  value_scales=vs64[inv], page_table=perm[None, :], **common)[0]
    assert torch.equal(got, want)
