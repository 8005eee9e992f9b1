"""CPU oracle of the MLA latent-cache path. TEST INFRASTRUCTURE: only tests, the smoke check and
the benchmark's CPU baseline may import it; the product never does.

PARITY UNPINNED: OpenBitSys/BitDecoding-FP4 contains no MLA code (src/nvfp4_vllm/backend.py:102
forwards ``use_mla`` and nothing consumes it), so there is no reference output or golden vector
to pin this against. What is pinned is every building block: the NVFP4 quantizer
(:func:`oracle.nvfp4_oracle.quantize_last_axis`, checked against the reference's vectors), the
page byte layouts (the 64-token layouts of :mod:`oracle.nvfp4_oracle`) and the softmax with its
FP4 probability operand (:func:`oracle.nvfp4_oracle.online_attention`, the restatement of
src/nvfp4_decode_kernel/reference.py:528-641). This module only composes them:

    score[h, t] = q_latent_fp4[h] . latent_k[t] + q_rope[h] . rope[t]
    out[h]      = online softmax over 128-token steps, newest first, of P_fp4 . latent_v

with ``latent_k`` the copy quantized along channels and ``latent_v`` the copy quantized along the
tokens of each 64-token page.
"""

from __future__ import annotations

import torch

from . import nvfp4_oracle as base

PAGE_TOKENS = 64
LATENT = 512
ROPE = 64
STEP = 128


def quantize_pages(latent: torch.Tensor, key_scale_mode: str = "amax6", value_scale_mode: str = "amax6"):
    """BF16 ``[pages, 64, 512]`` -> the four byte regions of the cache as the GQA page layouts give
    them for four 128-channel pseudo heads: K codes ``[pages,64,4,64]`` (logical view), K scales
    ``[pages,4,512]``, V codes ``[pages,4,128,32]``, V scales ``[pages,4,512]``."""
    pages = latent.shape[0]
    heads = latent.reshape(pages, PAGE_TOKENS, LATENT // 128, 128)
    key_codes, key_scales = base.quantize_key_pages(heads, key_scale_mode)
    value_codes, value_scales = base.quantize_value_pages(heads, value_scale_mode)
    return key_codes, key_scales, value_codes, value_scales


def rope_page_bytes(rope: torch.Tensor) -> torch.Tensor:
    """BF16 ``[pages, 64, 64]`` -> u8 ``[pages, 8192]``: token t's 128 bytes with 16-byte chunk j at
    position ``j ^ (t & 7)``."""
    pages = rope.shape[0]
    raw = rope.contiguous().view(torch.uint8).reshape(pages, PAGE_TOKENS, 128)
    key = (torch.arange(PAGE_TOKENS) & 7)[None, :]
    return base._place_chunks(raw, key).reshape(pages, 8192)


def quantize_query(q_latent: torch.Tensor, scale_mode: str = "amax6"):
    """BF16 ``[rows, heads, 512]`` -> (codes u8 ``[rows,heads,256]``, scale bytes ``[rows,heads,32]``,
    round-trip values FP32)."""
    codes, scales = base.quantize_last_axis(q_latent.float(), scale_mode)
    return base.pack_nibbles(codes), base.e4m3_bytes(scales), base.dequantize_last_axis(codes, scales)


def decode_reference(*, q_values: torch.Tensor, q_rope: torch.Tensor, key_codes, key_scales, value_codes,
                     value_scales, rope: torch.Tensor, page_table: torch.Tensor, seq_lens, softmax_scale: float,
                     p_mode: str = "amax2_or_amax6_c8", tau: float = base.DEFAULT_P_TAU, num_splits: int = 1):
    """``q_values`` FP32 ``[rows, heads, 512]`` (the FP4 query's values), ``q_rope`` BF16
    ``[rows, heads, 64]``, cache regions indexed by physical page, ``rope`` BF16 ``[pages, 64, 64]``.
    Returns ``(out BF16 [rows,heads,512], partial_out [parts,rows,heads,512], partial_lse)``."""
    rows, heads, _ = q_values.shape
    partial_out = torch.zeros(num_splits, rows, heads, LATENT)
    partial_lse = torch.full((num_splits, rows, heads), -torch.inf)
    for row in range(rows):
        length = int(seq_lens[row])
        entries = -(-length // PAGE_TOKENS)
        steps = -(-length // STEP)
        if steps == 0:
            continue
        ids = page_table[row, :entries].long()
        if entries % 2:  # the kernel walks the last page twice; its second half is masked
            ids = torch.cat([ids, ids[-1:]])
        latent_k = base.dequantize_key_pages(key_codes[ids], key_scales[ids]).reshape(-1, LATENT)
        latent_v = base.dequantize_value_pages(value_codes[ids], value_scales[ids]).reshape(-1, LATENT)
        rope_k = rope[ids].float().reshape(-1, ROPE)
        scores = q_values[row].float() @ latent_k.T + q_rope[row].float() @ rope_k.T
        scores[:, length:] = -torch.inf
        chunk = -(-steps // num_splits)
        for part in range(num_splits):
            first, last = min(part * chunk, steps), min((part + 1) * chunk, steps)
            if last <= first:
                continue
            blocks = [(scores[:, s * STEP:(s + 1) * STEP], latent_v[s * STEP:(s + 1) * STEP], "fp4")
                      for s in range(last - 1, first - 1, -1)]
            out, lse = base.online_attention(blocks, softmax_scale=softmax_scale, p_mode=p_mode, tau=tau)
            partial_out[part, row] = out
            partial_lse[part, row] = lse
    if num_splits == 1:
        return partial_out[0].to(torch.bfloat16), partial_out, partial_lse
    return base.combine_partials(partial_out, partial_lse), partial_out, partial_lse


def plain_attention(q_latent: torch.Tensor, q_rope: torch.Tensor, latent: torch.Tensor, rope: torch.Tensor,
                    softmax_scale: float) -> torch.Tensor:
    """Exact FP32 attention of one row from the unquantized tensors: ``[heads,512]`` out."""
    scores = (q_latent.float() @ latent.float().T + q_rope.float() @ rope.float().T) * softmax_scale
    return torch.softmax(scores, dim=-1) @ latent.float()
