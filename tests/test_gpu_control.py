"""The CUDA control-plane kernels (through the C ABI) against the golden vectors taken from the
reference's Triton kernels. Integer work: bit-exact, step by step, state included."""

from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GOLDEN = np.load(Path(__file__).parent / "golden" / "control_vectors.npz")
OUTPUTS = ("row_to_slot", "seqused_sink", "seqused_fp4", "seqused_residual", "promotion_source_tokens",
           "promotion_pages", "slot_keys", "slot_last_seq", "slot_last_seen")


def _dev(array, dtype=torch.int32):
    return torch.from_numpy(np.ascontiguousarray(array)).to(dtype).cuda()


@pytest.mark.parametrize("name", ["scripted", "random"])
def test_control_step_replays_reference(name):
    import bdfp4

    slots, max_tokens = 8, 2048
    state = dict(
        slot_keys=torch.full((slots,), -1, dtype=torch.int32, device="cuda"),
        slot_last_seq=torch.full((slots,), -1, dtype=torch.int32, device="cuda"),
        slot_last_seen=torch.full((slots,), -1, dtype=torch.int64, device="cuda"),
        step=torch.zeros(1, dtype=torch.int64, device="cuda"),
        row_to_slot=torch.full((slots,), -1, dtype=torch.int32, device="cuda"),
        token_to_slot=torch.full((max_tokens,), -1, dtype=torch.int32, device="cuda"),
        seqused_sink=torch.zeros(slots, dtype=torch.int32, device="cuda"),
        seqused_fp4=torch.zeros(slots, dtype=torch.int32, device="cuda"),
        seqused_residual=torch.zeros(slots, dtype=torch.int32, device="cuda"),
        promotion_source_tokens=torch.zeros(slots, dtype=torch.int32, device="cuda"),
        promotion_pages=torch.full((slots,), -1, dtype=torch.int32, device="cuda"),
        error_code=torch.zeros(1, dtype=torch.int32, device="cuda"),
    )
    stream = bdfp4.current_stream(torch.device("cuda"))
    for s in range(GOLDEN[f"{name}_num_reqs"].shape[0]):
        block_table = _dev(GOLDEN[f"{name}_block_table"][s])
        seq_lens = _dev(GOLDEN[f"{name}_seq_lens"][s])
        qsl = _dev(GOLDEN[f"{name}_query_start_loc"][s])
        a = bdfp4.ControlArgs()
        a.block_table, a.block_table_stride, a.block_table_columns = block_table.data_ptr(), block_table.stride(0), 6
        a.seq_lens, a.query_start_loc = seq_lens.data_ptr(), qsl.data_ptr()
        for key, tensor in state.items():
            setattr(a, key, tensor.data_ptr())
        a.num_reqs = int(GOLDEN[f"{name}_num_reqs"][s])
        a.num_actual_tokens = int(GOLDEN[f"{name}_num_tokens"][s])
        a.num_slots, a.sink_tokens = slots, 16
        bdfp4.control_step(a, stream)
        torch.cuda.synchronize()
        for key in OUTPUTS:
            assert np.array_equal(state[key].cpu().numpy(), GOLDEN[f"{name}_{key}"][s]), (name, s, key)
        assert int(state["error_code"].item()) == int(GOLDEN[f"{name}_error_code"][s][0]), (name, s)
        tokens = a.num_actual_tokens
        assert np.array_equal(state["token_to_slot"][:tokens].cpu().numpy(),
                              GOLDEN[f"{name}_token_to_slot"][s][:tokens])


def test_work_table_and_tail_reset():
    import bdfp4

    stream = bdfp4.current_stream(torch.device("cuda"))
    qsl, fp4, slot = _dev(GOLDEN["work_qsl"]), _dev(GOLDEN["work_fp4"]), _dev(GOLDEN["work_slot"])
    block_table = _dev(GOLDEN["work_block_table"])
    source = torch.full((12,), -7, dtype=torch.int32, device="cuda")
    destination = torch.full((12,), -7, dtype=torch.int32, device="cuda")
    bdfp4.work_table(qsl, fp4, slot, block_table, source, destination, 4, 3, stream)
    assert np.array_equal(source.cpu().numpy(), GOLDEN["work_source_tokens"])
    assert np.array_equal(destination.cpu().numpy(), GOLDEN["work_destination_pages"])

    layers, slots, tokens, heads, dim = 2, 4, 144, 2, 128
    tail_key = torch.ones(layers, slots, tokens, heads, dim, dtype=torch.bfloat16, device="cuda")
    tail_value = torch.full_like(tail_key, 2.0)
    bdfp4.tail_reset(tail_key, tail_value, qsl, _dev(GOLDEN["reset_seq_lens"]), slot, 4, stream)
    cleared_k = (tail_key.float().abs().sum(dim=(2, 3, 4)) == 0).cpu().numpy()
    cleared_v = (tail_value.float().abs().sum(dim=(2, 3, 4)) == 0).cpu().numpy()
    untouched = (tail_key.float().sum(dim=(2, 3, 4)) == tokens * heads * dim).cpu().numpy()
    assert np.array_equal(cleared_k, GOLDEN["reset_cleared_slots"])
    assert np.array_equal(cleared_v, GOLDEN["reset_cleared_slots"])
    assert np.array_equal(untouched, ~GOLDEN["reset_cleared_slots"])
