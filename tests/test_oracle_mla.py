"""CPU checks of the MLA oracle's composition (no GPU): layouts invert, and the kernel-faithful
attention stays close to exact attention over the dequantized cache."""

import torch

from oracle import mla_oracle as oracle
from oracle import nvfp4_oracle as base


def _case(tokens, heads, seed):
    gen = torch.Generator().manual_seed(seed)
    latent = torch.randn(tokens, 512, generator=gen).to(torch.bfloat16)
    rope = torch.randn(tokens, 64, generator=gen).to(torch.bfloat16)
    q_latent = torch.randn(1, heads, 512, generator=gen).to(torch.bfloat16)
    q_rope = torch.randn(1, heads, 64, generator=gen).to(torch.bfloat16)
    return latent, rope, q_latent, q_rope


def test_rope_block_layout_is_an_involution():
    gen = torch.Generator().manual_seed(1)
    rope = torch.randn(3, 64, 64, generator=gen).to(torch.bfloat16)
    block = oracle.rope_page_bytes(rope)
    assert block.shape == (3, 8192)
    raw = rope.contiguous().view(torch.uint8).reshape(3, 64, 128)
    # token 5, chunk 2 sits at chunk position 2 ^ 5
    assert torch.equal(block.reshape(3, 64, 8, 16)[:, 5, 2 ^ 5], raw.reshape(3, 64, 8, 16)[:, 5, 2])
    again = base._place_chunks(block.reshape(3, 64, 128), (torch.arange(64) & 7)[None, :])
    assert torch.equal(again, raw)


def test_both_latent_copies_dequantize_to_the_latent():
    latent, _, _, _ = _case(128, 4, 2)
    kc, ks, vc, vs = oracle.quantize_pages(latent.reshape(2, 64, 512))
    k = base.dequantize_key_pages(kc, ks).reshape(128, 512)
    v = base.dequantize_value_pages(vc, vs).reshape(128, 512)
    for copy in (k, v):
        rel = (copy - latent.float()).abs().mean() / latent.float().abs().mean()
        assert float(rel) < 0.12


def test_decode_reference_tracks_exact_attention_and_splits_agree():
    tokens, heads = 300, 8
    latent, rope, q_latent, q_rope = _case(320, heads, 3)
    latent[tokens:] = 0
    rope[tokens:] = 0
    kc, ks, vc, vs = oracle.quantize_pages(latent.reshape(5, 64, 512))
    _, _, q_values = oracle.quantize_query(q_latent)
    table = torch.arange(5, dtype=torch.int32)[None, :]
    args = dict(q_values=q_values, q_rope=q_rope, key_codes=kc, key_scales=ks, value_codes=vc, value_scales=vs,
                rope=rope.reshape(5, 64, 64), page_table=table, seq_lens=torch.tensor([tokens]),
                softmax_scale=576 ** -0.5)
    out, _, _ = oracle.decode_reference(**args)
    exact = oracle.plain_attention(q_latent[0], q_rope[0], latent[:tokens], rope[:tokens], 576 ** -0.5)
    assert float((out[0].float() - exact).abs().mean() / exact.abs().mean()) < 0.2
    split, partial_out, partial_lse = oracle.decode_reference(**args, num_splits=2)
    assert partial_out.shape == (2, 1, heads, 512) and torch.isfinite(partial_lse).all()
    assert float((split.float() - out.float()).abs().max()) < 2e-2
