"""CPU oracle of the device-side serving metadata (slot table, work table, tail reset).

TEST INFRASTRUCTURE ONLY: nothing in the product package imports this. It restates the reference's
Triton kernels (src/nvfp4_vllm/control.py:140-370, src/nvfp4_vllm/write.py:28-128 of
OpenBitSys/BitDecoding-FP4) in plain Python loops. Parity is pinned: the vectors of
``tests/golden/control_vectors.npz`` come from those kernels run under Triton's CPU interpreter
(``tests/golden/make_control_golden.py``) and ``tests/test_control_golden.py`` checks this model
against them.
"""

from __future__ import annotations

import numpy as np

PAGE = 128
FREE_KEY, NULL_BLOCK, INACTIVE = -1, 0, -1
ERRORS = {
    1: "a prompt arrived split across steps",
    2: "a row with history matched no slot",
    4: "a matched slot's length does not continue",
    8: "a row needing a slot found none free",
    16: "two live rows share a physical block",
    32: "a promotion column is past the block table",
}


class SlotTable:
    """Persistent state of the control plane (src/nvfp4_vllm/control.py:398-461)."""

    def __init__(self, num_slots: int, max_tokens: int, sink_tokens: int = 16):
        self.num_slots, self.sink = num_slots, sink_tokens
        self.slot_keys = np.full(num_slots, FREE_KEY, np.int32)
        self.slot_last_seq = np.full(num_slots, -1, np.int32)
        self.slot_last_seen = np.full(num_slots, -1, np.int64)
        self.step = 0
        self.row_to_slot = np.full(num_slots, INACTIVE, np.int32)
        self.seqused_sink = np.zeros(num_slots, np.int32)
        self.seqused_fp4 = np.zeros(num_slots, np.int32)
        self.seqused_residual = np.zeros(num_slots, np.int32)
        self.promotion_source_tokens = np.zeros(num_slots, np.int32)
        self.promotion_pages = np.full(num_slots, INACTIVE, np.int32)
        self.token_to_slot = np.full(max_tokens, INACTIVE, np.int32)
        self.error_code = 0

    def prepare(self, block_table, seq_lens, query_start_loc, num_reqs: int, num_tokens: int) -> None:
        """One step (src/nvfp4_vllm/control.py:140-370)."""
        n = self.num_slots
        self.step += 1
        keys = [int(block_table[i, 0]) if i < num_reqs else FREE_KEY for i in range(n)]
        seqs = [int(seq_lens[i]) if i < num_reqs else 0 for i in range(n)]
        begin = [int(query_start_loc[i]) if i < num_reqs else 0 for i in range(n)]
        end = [int(query_start_loc[i + 1]) if i < num_reqs else 0 for i in range(n)]
        live = [i < num_reqs and seqs[i] > 0 and keys[i] != NULL_BLOCK for i in range(n)]
        computed = [seqs[i] - (end[i] - begin[i]) for i in range(n)]
        matched = []
        for i in range(n):
            hit = [j for j in range(n) if live[i] and self.slot_keys[j] == keys[i]]
            matched.append(hit[0] if hit else n)
        claimed = [any(matched[i] == j for i in range(n)) for j in range(n)]
        needs = [live[i] and matched[i] == n for i in range(n)]
        free = [not claimed[j] for j in range(n)]
        order = sorted((j for j in range(n) if free[j]), key=lambda j: (int(self.slot_last_seen[j]), j))
        slots, errors, rank = [], 0, 0
        for i in range(n):
            if not live[i]:
                slots.append(INACTIVE)
                continue
            if matched[i] < n:
                slots.append(matched[i])
                if int(self.slot_last_seq[matched[i]]) != computed[i] and computed[i] > 0:
                    errors |= 4
            else:
                if rank < len(order):
                    slots.append(order[rank])
                else:
                    slots.append(0)
                    errors |= 8
                rank += 1
                if computed[i] > 0:
                    errors |= 2
            if end[i] - begin[i] > 1 and computed[i] > 0:
                errors |= 1
            if sum(1 for r in range(n) if live[r] and keys[r] == keys[i]) > 1:
                errors |= 16
        for j in range(n):
            owners = [i for i in range(n) if live[i] and slots[i] == j]
            if owners:
                self.slot_keys[j] = keys[owners[0]]
                self.slot_last_seq[j] = seqs[owners[0]]
                self.slot_last_seen[j] = self.step
        for i in range(n):
            seq = seqs[i] if live[i] else 0
            fp4 = ((seq - 1) // PAGE) * PAGE if seq > 0 else 0
            self.row_to_slot[i] = slots[i]
            self.seqused_sink[i] = min(seq, self.sink)
            self.seqused_fp4[i] = fp4
            self.seqused_residual[i] = seq - fp4
            column = fp4 // PAGE
            crossing = live[i] and seq > 0 and seq % PAGE == 0
            in_bounds = column < block_table.shape[1]
            if crossing and not in_bounds:
                errors |= 32
            self.promotion_source_tokens[i] = slots[i] * (PAGE + self.sink) if live[i] else 0
            self.promotion_pages[i] = int(block_table[i, column]) if crossing and in_bounds else INACTIVE
        self.error_code |= errors
        for token in range(num_tokens):
            self.token_to_slot[token] = sum(
                slots[r] for r in range(num_reqs) if live[r] and begin[r] <= token < end[r])


def work_table(query_start_loc, seqused_fp4, row_to_slot, block_table, num_reqs: int, columns: int):
    """(source_tokens, destination_pages) of the quantizer's grid (src/nvfp4_vllm/write.py:28-78)."""
    source = np.zeros(num_reqs * columns, np.int32)
    destination = np.full(num_reqs * columns, -1, np.int32)
    for row in range(num_reqs):
        start, end = int(query_start_loc[row]), int(query_start_loc[row + 1])
        writes = end - start > 1 and int(row_to_slot[row]) >= 0
        for column in range(columns):
            source[row * columns + column] = start + column * PAGE
            if writes and column < int(seqused_fp4[row]) // PAGE:
                destination[row * columns + column] = int(block_table[row, column])
    return source, destination


def rows_to_reset(query_start_loc, seq_lens, row_to_slot, num_reqs: int):
    """Slots whose tail pages a step clears: rows starting a request (src/nvfp4_vllm/write.py:81-128)."""
    cleared = set()
    for row in range(num_reqs):
        brought = int(query_start_loc[row + 1]) - int(query_start_loc[row])
        if int(row_to_slot[row]) >= 0 and int(seq_lens[row]) <= brought:
            cleared.add(int(row_to_slot[row]))
    return cleared
