"""The CPU oracle against vectors produced by the reference's own reference.py
(tests/golden/make_golden.py). Bit-exact for codes, scale bytes and winners; round-trip
values compare exactly because both sides multiply the same code by the same scale."""

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as oracle


def t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("mode", ["amax6", "four_six", "four_six_sixhalf"])
def test_block_scale_quantizer(golden, mode):
    x = t(golden["quant_x"])
    groups = x.reshape(x.shape[0], 8, 16)
    codes, scale, winner = oracle.quantize_groups(groups, mode)
    assert torch.equal(oracle.e4m3_bytes(scale), t(golden[f"quant_scales_{mode}"]))
    assert torch.equal(winner.to(torch.int8), t(golden[f"quant_winner_{mode}"]))
    want_codes = t(golden[f"quant_codes_{mode}"]).reshape(codes.shape)
    # The reference's CPU model encodes a negative value that rounds to zero as 8 but -0.0 as 0;
    # the hardware conversion (and this oracle) keeps the sign bit in both cases.
    same = (codes == want_codes) | ((codes & 7) == 0) & ((want_codes & 7) == 0)
    assert bool(same.all())
    values = oracle.dequantize_last_axis(codes.reshape(x.shape), scale)
    assert torch.equal(values, t(golden[f"quant_values_{mode}"]))


def test_e2m1_rounding(golden):
    x = t(golden["e2m1_x"])
    codes = oracle.e2m1_codes(x)
    assert torch.equal(codes, t(golden["e2m1_codes"]))
    assert torch.equal(oracle.e2m1_decode(codes), t(golden["e2m1_round"]))


def test_hadamard_and_two_term(golden):
    x = t(golden["had_x"])
    y = oracle.hadamard_rotate(x)
    assert torch.equal(y, t(golden["had_y"]))
    q = oracle.quantize_query(y.to(torch.bfloat16)[None].reshape(1, 6, 128), heads_kv=6, scale_mode="four_six", terms=2)
    # the two-term golden is taken from the FP32 rotated values, not their BF16 rounding
    codes, scales = oracle.quantize_last_axis(y, "four_six")
    first = oracle.dequantize_last_axis(codes, scales)
    assert torch.equal(first, t(golden["two_term_first"]))
    codes2, scales2 = oracle.quantize_last_axis(y - first, "four_six")
    assert torch.equal(oracle.dequantize_last_axis(codes2, scales2), t(golden["two_term_second"]))
    assert q["codes"][0].shape == (1, 1, 6, 64)


def test_value_token_axis(golden):
    v = t(golden["vtok_x"])  # [300, 2, 32]
    want = t(golden["vtok_y"])
    pages = v[:256].reshape(2, 128, 2, 32).permute(0, 2, 3, 1)  # [pages,H,ch,tok]
    codes, scales = oracle.quantize_last_axis(pages, "four_six")
    got = oracle.dequantize_last_axis(codes, scales).permute(0, 3, 1, 2).reshape(256, 2, 32)
    assert torch.equal(got[16:], want[16:256])
    assert torch.equal(want[256:], v[256:])


@pytest.mark.parametrize("mode", ["amax6", "amax2_or_amax6", "amax2_or_amax6_c8"])
def test_probability_operand(golden, mode):
    p = t(golden["p_x"])
    tau = float(golden["p_tau"])
    if mode.endswith("_c8"):
        got = oracle.probability_quantize(p * 8.0, "amax2_or_amax6", tau) * 0.125
    else:
        got = oracle.probability_quantize(p, mode, tau)
    assert torch.equal(got, t(golden[f"p_y_{mode}"]))


def _blocks(golden, values_fp4):
    scores = t(golden["attn_scores"]) / (128 ** -0.5) * (128 ** -0.5)  # raw scores; scale applied inside
    vals = t(golden["attn_values"])
    heads, tokens = scores.shape
    per_head = []
    for h in range(heads):
        per_head.append(oracle.kernel_order_blocks(
            scores_fp4=scores[h:h + 1, :384], values_fp4=values_fp4[:384, h], fp4_tokens=384,
            scores_tail=scores[h:h + 1, 384:], values_tail=vals[384:, h], tail_tokens=tokens - 384,
            scores_sink=scores[h:h + 1, :16], values_sink=vals[:16, h], sink_tokens=16))
    return per_head


@pytest.mark.parametrize("threshold", [0.0, 8.0])
def test_online_softmax_amax6(golden, threshold):
    fp4 = t(golden["attn_values_fp4"])
    want = t(golden[f"attn_out_amax6_thr{int(threshold)}"])
    for h, blocks in enumerate(_blocks(golden, fp4)):
        out, _ = oracle.online_attention(blocks, softmax_scale=128 ** -0.5, p_mode="amax6",
                                         rescale_threshold=threshold)
        # same arithmetic, different exp/sum association: agreement to FP32 rounding
        torch.testing.assert_close(out[0], want[h], rtol=2e-5, atol=2e-6)


def test_online_softmax_c8(golden):
    fp4 = t(golden["attn_values_fp4"])
    want = t(golden["attn_out_c8_p_and_v"])
    for h, blocks in enumerate(_blocks(golden, fp4)):
        out, lse = oracle.online_attention(blocks, softmax_scale=128 ** -0.5, p_mode="amax2_or_amax6_c8",
                                           rescale_threshold=0.0)
        torch.testing.assert_close(out[0], want[h], rtol=2e-5, atol=2e-6)
        scores = t(golden["attn_scores"])[h] * 128 ** -0.5
        torch.testing.assert_close(lse[0], torch.logsumexp(scores, dim=0), rtol=1e-5, atol=1e-5)


def test_sequence_split(golden):
    for n, want in zip(golden["seq_lens"], golden["seq_split"]):
        assert oracle.split_sequence_length(int(n)) == tuple(int(w) for w in want)
    for n, want in zip(golden["seq_lens"], golden["seq_split_sink4_page64"]):
        assert oracle.split_sequence_length(int(n), 4, 64) == tuple(int(w) for w in want)
