"""Generate the golden vectors under tests/golden/ from the reference's own CPU code.

Run in a container where OpenBitSys/BitDecoding-FP4 is mounted (see --reference):

    python tests/golden/make_golden.py [--reference <checkout of OpenBitSys/BitDecoding-FP4>]

It imports ``src/nvfp4_decode_kernel/reference.py`` (pure PyTorch, CPU), feeds it seeded
inputs, and stores inputs and outputs in ``tests/golden/reference_vectors.npz``. The tests
then check the repository's CPU oracle against these vectors without needing the reference.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch


def adversarial_rows() -> torch.Tensor:
    """Rows of 128 BF16-representable values that stress the scale search and the rounding."""
    rows = []
    rows.append(torch.zeros(128))
    rows.append(torch.full((128,), 1.0))
    rows.append(torch.full((128,), -3.0))
    # E2M1 midpoints under a scale of exactly 1 (amax 6): ties in both directions
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    rows.append(mids.repeat(8))
    # amax that flushes the E4M3 scale to zero, and one that is its smallest subnormal
    rows.append(torch.full((128,), 2.0 ** -12))
    rows.append(torch.cat([torch.full((64,), 6 * 2.0 ** -9), torch.full((64,), 3 * 2.0 ** -10)]))
    # amax past 448 * 6: the scale saturates
    rows.append(torch.cat([torch.full((16,), 4096.0), torch.linspace(-3000, 3000, 112)]))
    # one outlier per group, second-largest in the (4, 6) gap
    base = torch.tensor([6.0, 4.6, 1.1, -0.4, 0.2, 2.9, -3.4, 0.6, 5.1, -4.9, 0.9, 1.6, -2.1, 0.1, 0.3, -0.7])
    rows.append(base.repeat(8) * torch.tensor([1.0, 0.37, 17.0, 0.013, 250.0, 3.0, 0.11, 7.5]).repeat_interleave(16))
    # negative values that round to zero
    rows.append(torch.cat([torch.tensor([6.0]), torch.full((15,), -0.1)]).repeat(8))
    out = torch.stack(rows).to(torch.bfloat16).float()
    return out


def bf16_randn(gen, *shape):
    return torch.randn(*shape, generator=gen).to(torch.bfloat16).float()


def load_control(reference: Path):
    """``nvfp4_vllm/control.py`` as a stand-alone module (its package pulls in vLLM)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("_ref_control", reference / "src/nvfp4_vllm/control.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default="/root/reference")
    args = parser.parse_args()
    reference = Path(args.reference)
    sys.path.insert(0, str(reference / "src"))
    from nvfp4_decode_kernel import reference as ref  # noqa: E402

    gen = torch.Generator().manual_seed(20240)
    out: dict[str, np.ndarray] = {}

    # 1. block-scale quantizer: adversarial rows + N(0,1) rows with lognormal outlier channels
    rand = bf16_randn(gen, 40, 128)
    outliers = torch.randperm(128, generator=gen)[:4]
    rand[:, outliers] *= torch.exp(1.5 * torch.randn(4, generator=gen))
    rand = rand.to(torch.bfloat16).float()
    x = torch.cat([adversarial_rows(), rand])
    out["quant_x"] = x.numpy()
    for mode in ("amax6", "four_six", "four_six_sixhalf"):
        values, scales, winner = ref.nvfp4_quantize(x, scale_mode=mode)
        out[f"quant_values_{mode}"] = values.numpy()
        out[f"quant_scales_{mode}"] = scales.view(torch.uint8).numpy()
        out[f"quant_winner_{mode}"] = winner.numpy().astype(np.int8)
        groups = x.reshape(x.shape[0], 8, 16)
        scale_f = scales.float()[..., None]
        out[f"quant_codes_{mode}"] = ref.e2m1_codes(groups * (1.0 / (scale_f + 1.0e-30))).reshape(x.shape).numpy()

    # 2. rounding primitives
    grid = torch.cat([torch.linspace(-7, 7, 281), torch.tensor(ref._E2M1_MIDPOINTS), -torch.tensor(ref._E2M1_MIDPOINTS)])
    out["e2m1_x"] = grid.numpy()
    out["e2m1_round"] = ref.round_e2m1(grid).numpy()
    out["e2m1_codes"] = ref.e2m1_codes(grid).numpy()

    # 3. Hadamard and the two-term query
    q = bf16_randn(gen, 6, 128)
    out["had_x"] = q.numpy()
    out["had_y"] = ref.hadamard_rotate(q).numpy()
    first, second = ref.nvfp4_two_term(ref.hadamard_rotate(q), scale_mode="four_six")
    out["two_term_first"] = first.numpy()
    out["two_term_second"] = second.numpy()

    # 4. V token-axis round trip
    tokens, heads = 300, 2
    v = bf16_randn(gen, tokens, heads, 32)
    out["vtok_x"] = v.numpy()
    out["vtok_y"] = ref.value_token_axis_round_trip(v, fp4_tokens=256, sink_tokens=16, scale_mode="four_six").numpy()

    # 5. P operand
    p = torch.rand(4, 128, generator=gen) ** 6
    p[0, :16] = 0.0
    p[1, 16:32] *= 1.0e-3
    out["p_x"] = p.numpy()
    for mode in ("amax6", "amax2_or_amax6", "amax2_or_amax6_c8"):
        values, _ = ref.nvfp4_probability_quantize(p, scale_mode=mode)
        out[f"p_y_{mode}"] = values.numpy()
    out["p_tau"] = np.float32(ref.P_SMALL_GROUP_AMAX)

    # 6. online softmax in kernel order
    heads_q, tokens = 4, 16 + 3 * 128 + 37
    scores = torch.randn(heads_q, tokens, generator=gen) * 6.0
    scores[1, 200] = 80.0  # a late, large score: exercises the stale-maximum threshold
    vals = bf16_randn(gen, tokens, heads_q, 16)
    fp4_vals = ref.value_token_axis_round_trip(vals, fp4_tokens=384, sink_tokens=16, scale_mode="amax6")
    out["attn_scores"] = scores.numpy()
    out["attn_values"] = vals.numpy()
    out["attn_values_fp4"] = fp4_vals.numpy()
    for threshold in (0.0, 8.0):
        o = ref.online_softmax_pv(scores, fp4_vals, fp4_tokens=384, quantize_probabilities=True,
                                  sink_tokens=16, rescale_threshold=threshold, softmax_scale=128 ** -0.5)
        out[f"attn_out_amax6_thr{int(threshold)}"] = o.numpy()
    factors = ref.online_softmax_pv_factors(scores, vals, fp4_vals, fp4_tokens=384, sink_tokens=16,
                                            softmax_scale=128 ** -0.5,
                                            probability_scale_mode="amax2_or_amax6_c8")
    out["attn_out_c8_p_and_v"] = factors["p_and_v"].numpy()
    out["attn_out_c8_reference"] = factors["reference"].numpy()

    # 7. sequence-length split
    control = load_control(reference)
    lens = [0, 1, 15, 16, 17, 127, 128, 129, 255, 256, 257, 4096, 65536]
    out["seq_lens"] = np.array(lens, dtype=np.int64)
    out["seq_split"] = np.array([control.split_sequence_length(n) for n in lens], dtype=np.int64)
    out["seq_split_sink4_page64"] = np.array(
        [control.split_sequence_length(n, sink_tokens=4, page_size=64) for n in lens], dtype=np.int64)

    # 8. host split policies (pure Python; the modules that hold two of them import GPU-only
    #    packages, so only the function's own source is executed)
    import ast
    import math as _math

    def extract(path: Path, name: str):
        tree = ast.parse(path.read_text())
        node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name)
        namespace = {"math": _math, "MAX_DECODE_SPLITS": 32}
        exec(compile(ast.Module([node], []), str(path), "exec"), namespace)
        return namespace[name]

    ref_num_splits = extract(reference / "src/nvfp4_vllm/builder.py", "decode_num_splits")
    ref_heuristic = extract(reference / "src/nvfp4_decode_kernel/_decode.py", "split_k_heuristic")
    from nvfp4_decode_kernel.interface import split_partial_count as ref_partial_count

    rows_grid = [1, 2, 3, 4, 7, 8, 16, 31, 32, 64, 128]
    out["policy_decode_num_splits"] = np.array(
        [(r, h, sms, ref_num_splits(r, h, sms)) for r in rows_grid for h in (1, 2, 4, 8) for sms in (132, 148)],
        dtype=np.int64)
    out["policy_split_k_heuristic"] = np.array(
        [(r, h, pages, 148, ref_heuristic(r, h, pages, sms=148))
         for r in rows_grid for h in (1, 4, 8) for pages in (1, 2, 7, 64, 511, 1023)], dtype=np.int64)
    out["policy_split_partial_count"] = np.array(
        [(r, h, s, int(res), 148, ref_partial_count(r, h, s, residual=res, sms=148))
         for r in (1, 4, 16, 64) for h in (1, 8) for s in (1, 2, 4, 9) for res in (False, True)], dtype=np.int64)

    target = Path(__file__).resolve().parent / "reference_vectors.npz"
    np.savez_compressed(target, **out)
    print(f"wrote {target} ({target.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    main()
