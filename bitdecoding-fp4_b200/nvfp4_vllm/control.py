"""Device-side slot table: which BF16 tail slot each batch row owns, and each row's lengths.

Keeps the names of src/nvfp4_vllm/control.py of OpenBitSys/BitDecoding-FP4 (``ControlPlane``,
``ControlOutputs``, ``split_sequence_length``, the error flags); the single-CTA kernel is
``bdfp4_control_step`` (CUDA) instead of Triton. A request is identified by the physical block
holding its first page (column 0 of its block-table row), which is fixed for its life; nothing
is read back to the host on a step.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

import bdfp4
from nvfp4_decode_kernel.interface import SINK_TOKENS

PAGE_SIZE = 128
TAIL_BUFFER_TOKENS = PAGE_SIZE + SINK_TOKENS
MAX_SUPPORTED_SLOTS = 128
FREE_KEY = -1
NULL_BLOCK = 0
INACTIVE_ROW = -1

ERR_CONTINUATION_PREFILL = 1
ERR_SLOT_LOST = 2
ERR_STALE_SLOT_HISTORY = 4
ERR_NO_FREE_SLOT = 8
ERR_DUPLICATE_KEY = 16
ERR_PROMOTION_COLUMN = 32
ERROR_NAMES = {
    ERR_CONTINUATION_PREFILL: "a prompt arrived split across steps",
    ERR_SLOT_LOST: "a row with history matched no slot",
    ERR_STALE_SLOT_HISTORY: "a matched slot's length does not continue",
    ERR_NO_FREE_SLOT: "a row needing a slot found none free",
    ERR_DUPLICATE_KEY: "two live rows share a physical block",
    ERR_PROMOTION_COLUMN: "a promotion column is past the block table",
}


def split_sequence_length(sequence_length: int, *, sink_tokens: int = SINK_TOKENS,
                          page_size: int = PAGE_SIZE) -> tuple[int, int, int]:
    """(sink, fp4, residual) token counts of a sequence. The sink overlays the unchanged page grid
    (page zero later holds a masked duplicate), so the three need not sum to the length."""
    if sequence_length < 0:
        raise ValueError(f"sequence_length must be nonnegative, got {sequence_length}")
    if sink_tokens < 0:
        raise ValueError(f"sink_tokens must be nonnegative, got {sink_tokens}")
    if page_size < 1:
        raise ValueError(f"page_size must be positive, got {page_size}")
    fp4 = ((sequence_length - 1) // page_size) * page_size if sequence_length else 0
    return min(sequence_length, sink_tokens), fp4, sequence_length - fp4


@dataclass(frozen=True)
class ControlOutputs:
    """Views into the control plane's scratch, valid until the next step; device-only."""

    row_to_slot: torch.Tensor
    token_to_slot: torch.Tensor
    seqused_sink: torch.Tensor  # full width: a captured decode sees one stable-shape tensor
    seqused_fp4: torch.Tensor
    seqused_residual: torch.Tensor
    promotion_source_tokens: torch.Tensor  # full width: promotion's grid is a constant of the engine
    promotion_pages: torch.Tensor
    error_code: torch.Tensor


class ControlPlaneError(RuntimeError):
    """An invariant the slot table reported through ``error_code``."""


class ControlPlane:
    """Slot table and per-step scratch of one engine, allocated once at the high-water mark."""

    def __init__(self, *, max_num_seqs: int, max_num_batched_tokens: int, device, page_size: int = PAGE_SIZE):
        if max_num_seqs < 1:
            raise ValueError(f"max_num_seqs must be positive, got {max_num_seqs}")
        if max_num_seqs > MAX_SUPPORTED_SLOTS:
            raise ValueError(
                f"max_num_seqs={max_num_seqs} exceeds the validated {MAX_SUPPORTED_SLOTS}-slot control-plane ceiling"
            )
        if max_num_batched_tokens < max_num_seqs:
            raise ValueError(
                f"max_num_batched_tokens ({max_num_batched_tokens}) must cover one token per row ({max_num_seqs})"
            )
        if page_size != PAGE_SIZE:
            raise ValueError(f"the control kernel is built for {PAGE_SIZE}-token pages, got {page_size}")
        self.num_slots = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.page_size = page_size
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())

        def slots(dtype, fill):
            return torch.full((self.num_slots,), fill, dtype=dtype, device=self.device)

        self.slot_keys = slots(torch.int32, FREE_KEY)
        self.slot_last_seq = slots(torch.int32, -1)  # -1 is no reachable computed-token count
        self.slot_last_seen = slots(torch.int64, -1)
        self.step = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.row_to_slot = slots(torch.int32, INACTIVE_ROW)
        self.seqused_sink = slots(torch.int32, 0)
        self.seqused_fp4 = slots(torch.int32, 0)
        self.seqused_residual = slots(torch.int32, 0)
        self.promotion_source_tokens = slots(torch.int32, 0)
        self.promotion_pages = slots(torch.int32, INACTIVE_ROW)
        self.error_code = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.token_to_slot = torch.full((max_num_batched_tokens,), INACTIVE_ROW, dtype=torch.int32,
                                        device=self.device)

    def reset(self) -> None:
        """Forget every slot. Only valid when no request is in flight."""
        self.slot_keys.fill_(FREE_KEY)
        self.slot_last_seq.fill_(-1)
        self.slot_last_seen.fill_(-1)
        self.step.zero_()
        self.error_code.zero_()

    def raise_for_errors(self) -> None:
        """Read the sticky error word (a host synchronisation) and raise if anything was reported."""
        code = int(self.error_code.item())
        if not code:
            return
        named = [text for bit, text in ERROR_NAMES.items() if code & bit]
        unknown = code & ~sum(ERROR_NAMES)
        if unknown:
            named.append(f"unrecognized flags {unknown:#x}")
        raise ControlPlaneError(f"the slot control plane reported error_code {code}: " + "; ".join(named))

    def prepare(self, *, block_table: torch.Tensor, seq_lens: torch.Tensor, query_start_loc: torch.Tensor,
                num_reqs: int, num_actual_tokens: int) -> ControlOutputs:
        """Advance the slot table by one step. ``seq_lens`` already counts this step's tokens; a row
        of length zero is padding; ``num_reqs`` / ``num_actual_tokens`` are host integers."""
        if block_table.ndim != 2:
            raise ValueError(f"block_table must be 2-D, got {block_table.ndim}-D")
        if num_reqs > self.num_slots:
            raise ValueError(f"{num_reqs} rows exceeds the {self.num_slots} tail slots")
        if num_actual_tokens > self.max_num_batched_tokens:
            raise ValueError(
                f"{num_actual_tokens} tokens exceeds the {self.max_num_batched_tokens} the scratch was sized for"
            )
        for name, tensor in (("block_table", block_table), ("seq_lens", seq_lens),
                             ("query_start_loc", query_start_loc)):
            if tensor.dtype is not torch.int32 or tensor.device != self.device:
                raise ValueError(f"{name} must be INT32 on {self.device}")
        if block_table.stride(1) != 1:
            raise ValueError("block_table rows must be contiguous")
        a = bdfp4.ControlArgs()
        a.block_table, a.block_table_stride = block_table.data_ptr(), block_table.stride(0)
        a.block_table_columns = block_table.shape[1]
        a.seq_lens, a.query_start_loc = seq_lens.data_ptr(), query_start_loc.data_ptr()
        for name in ("slot_keys", "slot_last_seq", "slot_last_seen", "step", "row_to_slot", "token_to_slot",
                     "seqused_sink", "seqused_fp4", "seqused_residual", "promotion_source_tokens",
                     "promotion_pages", "error_code"):
            setattr(a, name, getattr(self, name).data_ptr())
        a.num_reqs, a.num_actual_tokens = int(num_reqs), int(num_actual_tokens)
        a.num_slots, a.sink_tokens = self.num_slots, SINK_TOKENS
        bdfp4.control_step(a, bdfp4.current_stream(self.device))
        return ControlOutputs(
            row_to_slot=self.row_to_slot[:num_reqs],
            token_to_slot=self.token_to_slot[:num_actual_tokens],
            seqused_sink=self.seqused_sink,
            seqused_fp4=self.seqused_fp4[:num_reqs],
            seqused_residual=self.seqused_residual[:num_reqs],
            promotion_source_tokens=self.promotion_source_tokens,
            promotion_pages=self.promotion_pages,
            error_code=self.error_code,
        )
