"""Generate tests/golden/mxfp4_vectors.npz from the reference's own CPU code.

    python tests/golden/make_mxfp4_golden.py [--reference <checkout of OpenBitSys/BitDecoding-FP4>]

Imports ``src/nvfp4_decode_kernel/reference.py`` of OpenBitSys/BitDecoding-FP4 (pure PyTorch, CPU),
feeds ``mxfp4_quantize`` (three rules) and ``mxfp4_probability_quantize`` seeded and adversarial
inputs, and stores inputs and outputs. tests/test_oracle_mxfp4.py then checks the repository's
oracle against them without needing the reference.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch


def inputs() -> torch.Tensor:
    gen = torch.Generator().manual_seed(20240611)
    rows = [torch.randn(24, 128, generator=gen) * torch.exp(2.0 * torch.randn(24, 1, generator=gen))]
    special = []
    special.append(torch.zeros(128))
    special.append(torch.full((128,), 6.0))
    special.append(torch.full((128,), 6.0001))   # just past the E2M1 maximum on the OCP scale
    special.append(torch.full((128,), -7.9))
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    special.append(mids.repeat(8))               # E2M1 midpoints under scale 1
    special.append(mids.repeat(8) * 0.5)
    special.append(torch.full((128,), 2.0 ** -130))                 # below the smallest E8M0 scale times 0.5
    special.append(torch.cat([torch.full((32,), 3.0e38), torch.full((96,), 1.0e-30)]))  # the clamps
    base = torch.tensor([7.5, 4.6, 1.1, -0.4, 0.2, 2.9, -3.4, 0.6, 5.1, -4.9, 0.9, 1.6, -2.1, 0.1, 0.3, -0.7])
    special.append(base.repeat(8) * torch.tensor([1.0, 0.37, 17.0, 0.013]).repeat_interleave(32))
    rows.append(torch.stack(special))
    return torch.cat(rows).to(torch.bfloat16).float()


def probabilities() -> torch.Tensor:
    gen = torch.Generator().manual_seed(99)
    logits = torch.randn(16, 128, generator=gen) * torch.tensor([0.5, 1.0, 2.0, 4.0]).repeat(4)[:, None]
    p = torch.exp2(logits - logits.amax(dim=-1, keepdim=True))
    p[3, 40:] = 0.0
    p[7] = 0.0
    return torch.cat([p, 8.0 * p[:4]])


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default="/root/reference")
    args = parser.parse_args()
    sys.path.insert(0, str(Path(args.reference) / "src"))
    from nvfp4_decode_kernel import reference

    x = inputs()
    out = {"x": x.numpy()}
    for rule in ("ocp", "round_up", "search"):
        values, codes, winner = reference.mxfp4_quantize(x, rule)
        out[f"{rule}_values"] = values.numpy()
        out[f"{rule}_scale_bytes"] = codes.numpy()
        out[f"{rule}_winner"] = winner.numpy()
    p = probabilities()
    values, codes = reference.mxfp4_probability_quantize(p)
    out["p"] = p.numpy()
    out["p_values"] = values.numpy()
    out["p_scale_bytes"] = codes.numpy()
    target = Path(__file__).resolve().parent / "mxfp4_vectors.npz"
    np.savez_compressed(target, **out)
    print(f"wrote {target} ({target.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
