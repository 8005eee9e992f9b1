"""The control-plane oracle against vectors from the reference's Triton kernels (run under
Triton's CPU interpreter by tests/golden/make_control_golden.py). Integer work: exact."""

from pathlib import Path

import numpy as np
import pytest

from oracle import control_oracle

GOLDEN = np.load(Path(__file__).parent / "golden" / "control_vectors.npz")
OUTPUTS = ("row_to_slot", "seqused_sink", "seqused_fp4", "seqused_residual", "promotion_source_tokens",
           "promotion_pages", "slot_keys", "slot_last_seq", "slot_last_seen")


@pytest.mark.parametrize("name", ["scripted", "random"])
def test_slot_table_steps(name):
    steps = GOLDEN[f"{name}_num_reqs"].shape[0]
    table = control_oracle.SlotTable(8, 2048)
    for s in range(steps):
        num_reqs, tokens = int(GOLDEN[f"{name}_num_reqs"][s]), int(GOLDEN[f"{name}_num_tokens"][s])
        table.prepare(GOLDEN[f"{name}_block_table"][s], GOLDEN[f"{name}_seq_lens"][s],
                      GOLDEN[f"{name}_query_start_loc"][s], num_reqs, tokens)
        for key in OUTPUTS:
            assert np.array_equal(getattr(table, key), GOLDEN[f"{name}_{key}"][s]), (name, s, key)
        assert table.error_code == int(GOLDEN[f"{name}_error_code"][s][0]), (name, s)
        assert table.step == int(GOLDEN[f"{name}_step"][s][0])
        assert np.array_equal(table.token_to_slot[:tokens], GOLDEN[f"{name}_token_to_slot"][s][:tokens])


def test_scripted_scenario_raises_every_error_flag():
    assert int(GOLDEN["scripted_error_code"][-1][0]) == 1 | 2 | 4 | 16 | 32 or \
        int(GOLDEN["scripted_error_code"][-1][0]) & (1 | 2 | 16 | 32) == (1 | 2 | 16 | 32)


def test_work_table_and_tail_reset():
    source, destination = control_oracle.work_table(
        GOLDEN["work_qsl"], GOLDEN["work_fp4"], GOLDEN["work_slot"], GOLDEN["work_block_table"], 4, 3)
    assert np.array_equal(source, GOLDEN["work_source_tokens"])
    assert np.array_equal(destination, GOLDEN["work_destination_pages"])
    cleared = control_oracle.rows_to_reset(GOLDEN["work_qsl"], GOLDEN["reset_seq_lens"], GOLDEN["work_slot"], 4)
    want = GOLDEN["reset_cleared_slots"]  # [layers, slots]
    for layer in range(want.shape[0]):
        assert {int(s) for s in np.nonzero(want[layer])[0]} == cleared
