"""Golden vectors for the device-side control plane, from the reference's own Triton kernels.

    python tests/golden/make_control_golden.py [--reference <checkout of OpenBitSys/BitDecoding-FP4>]

Runs ``_control_kernel`` (src/nvfp4_vllm/control.py), ``_work_table_kernel`` and
``_tail_reset_kernel`` (src/nvfp4_vllm/write.py) of the mounted reference under Triton's CPU
interpreter (``TRITON_INTERPRET=1``) over a scripted and a seeded random sequence of serving
steps, and stores every step's inputs, outputs and slot-table state in
``tests/golden/control_vectors.npz``.
"""

from __future__ import annotations

import argparse
import importlib.util
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

SLOTS, COLUMNS, MAX_TOKENS = 8, 6, 2048


def load(reference: Path, name: str):
    spec = importlib.util.spec_from_file_location(f"_ref_{name}", reference / f"src/nvfp4_vllm/{name}.py")
    module = importlib.util.module_from_spec(spec)
    sys.modules[f"_ref_{name}"] = module
    spec.loader.exec_module(module)
    return module


def scripted_steps():
    """(rows) per step; a row is (key block, sequence length after the step, tokens this step)."""
    return [
        [(5, 300, 300), (9, 130, 130)],
        [(5, 301, 1), (9, 131, 1), (12, 128, 128)],
        [(5, 302, 1), (12, 129, 1), (3, 0, 0)],          # 9 sits out; a padding row keeps a stale block id
        [(5, 303, 1), (9, 132, 1), (12, 130, 1)],
        [(9, 50, 50), (5, 304, 1)],                       # block 9 recycled by a brand new request
        [(21, 10, 10), (22, 20, 20), (23, 30, 30), (24, 40, 40), (25, 50, 50), (26, 60, 60)],  # LRU reuse
        [(5, 305, 1), (5, 306, 1)],                       # two live rows share a block
        [(31, 400, 100)],                                 # continuation prefill with no slot: two errors
        [(0, 17, 1), (0, 9, 1)],                          # dummy batch over the null block
        [(21, 896, 886)],                                 # promotion column past the block table
        [(22, 256, 236), (23, 384, 354)],                 # tails that just filled: promotion targets
    ]


def random_steps(seed: int, count: int):
    rng = np.random.default_rng(seed)
    live: dict[int, int] = {}
    next_block = 100
    steps = []
    for _ in range(count):
        rows = []
        for key in list(live):
            roll = rng.random()
            if roll < 0.15:
                del live[key]
            elif roll < 0.85:
                live[key] += 1
                rows.append((key, live[key], 1))
        while len(rows) < SLOTS and len(live) < SLOTS and rng.random() < 0.5:
            length = int(rng.integers(1, 500))
            live[next_block] = length
            rows.append((next_block, length, length))
            next_block += 1
        rng.shuffle(rows)
        rows = [tuple(int(x) for x in r) for r in rows]
        decodes = [r for r in rows if r[2] == 1]
        prefills = [r for r in rows if r[2] != 1]
        steps.append(decodes + prefills)
    return steps


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default="/root/reference")
    args = parser.parse_args()
    reference = Path(args.reference)
    sys.path.insert(0, str(reference / "src"))
    control = load(reference, "control")
    sys.modules["nvfp4_vllm"] = type(sys)("nvfp4_vllm")
    sys.modules["nvfp4_vllm.control"] = control

    out: dict[str, np.ndarray] = {}
    for name, steps in (("scripted", scripted_steps()), ("random", random_steps(7, 40))):
        plane = control.ControlPlane(max_num_seqs=SLOTS, max_num_batched_tokens=MAX_TOKENS, device="cpu")
        records = {k: [] for k in (
            "block_table", "seq_lens", "query_start_loc", "num_reqs", "num_tokens", "row_to_slot", "token_to_slot",
            "seqused_sink", "seqused_fp4", "seqused_residual", "promotion_source_tokens", "promotion_pages",
            "error_code", "slot_keys", "slot_last_seq", "slot_last_seen", "step")}
        for rows in steps:
            block_table = torch.zeros(SLOTS, COLUMNS, dtype=torch.int32)
            seq_lens = torch.zeros(SLOTS, dtype=torch.int32)
            qsl = torch.zeros(SLOTS + 1, dtype=torch.int32)
            cursor = 0
            for r, (key, seq, tokens) in enumerate(rows):
                block_table[r, 0] = key
                block_table[r, 1:] = torch.arange(1, COLUMNS, dtype=torch.int32) + 1000 * (key + 1)
                seq_lens[r] = seq
                cursor += tokens
                qsl[r + 1] = cursor
            qsl[len(rows) + 1:] = cursor
            plane.prepare(block_table=block_table, seq_lens=seq_lens, query_start_loc=qsl, num_reqs=len(rows),
                          num_actual_tokens=cursor)
            snapshot = dict(
                block_table=block_table, seq_lens=seq_lens, query_start_loc=qsl,
                num_reqs=torch.tensor(len(rows)), num_tokens=torch.tensor(cursor), row_to_slot=plane.row_to_slot,
                token_to_slot=plane.token_to_slot, seqused_sink=plane.seqused_sink, seqused_fp4=plane.seqused_fp4,
                seqused_residual=plane.seqused_residual, promotion_source_tokens=plane.promotion_source_tokens,
                promotion_pages=plane.promotion_pages, error_code=plane.error_code, slot_keys=plane.slot_keys,
                slot_last_seq=plane.slot_last_seq, slot_last_seen=plane.slot_last_seen, step=plane.step)
            for key, value in snapshot.items():
                records[key].append(value.clone().numpy())
        for key, values in records.items():
            out[f"{name}_{key}"] = np.stack(values)

    # work table and tail reset on one mixed batch
    # write.py imports the CuTeDSL writer, which needs a GPU stack: load only its two Triton kernels
    source = (reference / "src/nvfp4_vllm/write.py").read_text()
    head = source.split("def reset_new_request_tails")[0]
    head = head.replace("from nvfp4_decode_kernel.quantize_kv_kernel import KVCacheWriter\n", "")
    head = head.replace("from .control import PAGE_SIZE", "PAGE_SIZE = 128")
    kernel_file = Path("/tmp/_ref_write_kernels.py")
    kernel_file.write_text(head)
    spec = importlib.util.spec_from_file_location("_ref_write_kernels", kernel_file)
    kernels = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(kernels)
    import triton

    qsl = torch.tensor([0, 1, 1 + 300, 1 + 300 + 128, 1 + 300 + 128 + 5], dtype=torch.int32)
    seqused_fp4 = torch.tensor([256, 256, 0, 0], dtype=torch.int32)
    row_to_slot = torch.tensor([3, 1, -1, 0], dtype=torch.int32)
    block_table = torch.arange(4 * COLUMNS, dtype=torch.int32).reshape(4, COLUMNS) + 50
    columns = 3
    source_tokens = torch.full((4 * columns,), -7, dtype=torch.int32)
    destination_pages = torch.full((4 * columns,), -7, dtype=torch.int32)
    kernels._work_table_kernel[(4,)](qsl, seqused_fp4, row_to_slot, block_table, block_table.stride(0),
                                     source_tokens, destination_pages, 4, columns, PAGE=128,
                                     BLOCK=triton.next_power_of_2(columns), num_warps=4)
    out["work_qsl"], out["work_fp4"], out["work_slot"] = qsl.numpy(), seqused_fp4.numpy(), row_to_slot.numpy()
    out["work_block_table"] = block_table.numpy()
    out["work_source_tokens"], out["work_destination_pages"] = source_tokens.numpy(), destination_pages.numpy()

    layers, slots, tokens, heads, dim = 2, 4, 144, 1, 8
    tail_key = torch.ones(layers, slots, tokens, heads, dim, dtype=torch.float32)
    tail_value = torch.full_like(tail_key, 2.0)
    seq_lens = torch.tensor([301, 300, 128, 9], dtype=torch.int32)  # rows 1..3 start a request this step
    kernels._tail_reset_kernel[(layers, 4)](tail_key, tail_value, tail_key.stride(0), tail_key.stride(1), qsl,
                                            seq_lens, row_to_slot, 4, WIDTH=heads * dim, TOKENS=tokens, num_warps=4)
    out["reset_seq_lens"] = seq_lens.numpy()
    out["reset_cleared_slots"] = (tail_key[:, :, 0, 0, 0] == 0).numpy()
    assert bool(((tail_key == 0) == (tail_value == 0)).all())

    target = Path(__file__).resolve().parent / "control_vectors.npz"
    np.savez_compressed(target, **out)
    print(f"wrote {target} ({target.stat().st_size} bytes)")


if __name__ == "__main__":
    main()
