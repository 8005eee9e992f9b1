"""The MXFP4 oracle against outputs of the reference's own mxfp4_quantize and
mxfp4_probability_quantize (tests/golden/mxfp4_vectors.npz, made by make_mxfp4_golden.py): values,
E8M0 bytes and the winning exponent bit-exact, for every rule. No GPU; MXFP4 has no kernel yet."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import mxfp4_oracle as mx

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def vectors():
    return np.load(ROOT / "tests" / "golden" / "mxfp4_vectors.npz")


@pytest.mark.parametrize("rule", mx.RULES)
def test_quantizer_matches_the_reference(vectors, rule):
    x = torch.from_numpy(vectors["x"])
    codes, scale_bytes, winner = mx.quantize_last_axis(x, rule)
    assert torch.equal(scale_bytes, torch.from_numpy(vectors[f"{rule}_scale_bytes"]))
    assert torch.equal(winner, torch.from_numpy(vectors[f"{rule}_winner"]))
    values = mx.dequantize_last_axis(codes, scale_bytes)
    want = torch.from_numpy(vectors[f"{rule}_values"])
    assert torch.equal(values, want)  # -0.0 == 0.0 here: the reference returns values, not codes


def test_search_is_never_worse_than_either_fixed_rule(vectors):
    x = torch.from_numpy(vectors["x"])
    errors = {}
    for rule in mx.RULES:
        codes, scale_bytes, _ = mx.quantize_last_axis(x, rule)
        difference = (mx.dequantize_last_axis(codes, scale_bytes) - x).reshape(-1, 32)
        errors[rule] = difference.double().square().sum(dim=-1)
    finite = torch.isfinite(errors["search"])
    assert (errors["search"][finite] <= errors["ocp"][finite] * (1 + 1e-6)).all()
    assert (errors["search"][finite] <= errors["round_up"][finite] * (1 + 1e-6)).all()


def test_probability_operand_matches_the_reference(vectors):
    p = torch.from_numpy(vectors["p"])
    values, scale_bytes = mx.probability_quantize(p)
    assert torch.equal(scale_bytes, torch.from_numpy(vectors["p_scale_bytes"]))
    assert torch.equal(values, torch.from_numpy(vectors["p_values"]))


def test_zero_group_and_clamps():
    zero = torch.zeros(1, 32)
    codes, scale_bytes, _ = mx.quantize_last_axis(zero, "search")
    assert int(scale_bytes) == 0 and int(codes.sum()) == 0  # exponent -127: E8M0 has no zero
    huge = torch.full((1, 32), 3.0e38)
    _, scale_bytes, _ = mx.quantize_last_axis(huge, "round_up")
    assert int(scale_bytes) <= 254
