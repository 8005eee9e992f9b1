"""GPU state one model's NVFP4 layers share for their whole lifetime (src/nvfp4_vllm/runtime.py of
OpenBitSys/BitDecoding-FP4): the BF16 sink + rolling-tail buffers, the carved cache views, the
query and split scratch, the key-shift sidecar and the writers built on them.

Created during the profile run, before the KV cache exists, so that the engine subtracts this
memory from the cache budget. Only the rotations the kernels fuse are built (``none`` and the
Sylvester ``hadamard``); ``block_hadamard_64`` is not.
"""

from __future__ import annotations

import os

import torch

from nvfp4_decode_kernel import RESIDUAL_ROW_TILE, split_partial_count
from nvfp4_decode_kernel.quantize_kv_kernel import KVCacheWriter
from nvfp4_decode_kernel.scale_mode import DEFAULT_SCALE_MODE, sf_vec_size

from . import layout
from .control import SINK_TOKENS, TAIL_BUFFER_TOKENS

PAGE_SIZE = 128
# Workers load the key-smoothing mean from this safetensors path: tensor ``key_shift`` of shape
# ``[num_layers, num_kv_heads, head_dim]`` in the model's original (unrotated) basis.
KEY_SHIFT_ENV = "NVFP4_KEY_SHIFT"


def sylvester_hadamard(order: int, device, dtype=torch.float64) -> torch.Tensor:
    """Normalised Sylvester Hadamard matrix of a power-of-two order."""
    matrix = torch.ones(1, 1, dtype=dtype, device=device)
    while matrix.shape[0] < order:
        matrix = torch.cat((torch.cat((matrix, matrix), 1), torch.cat((matrix, -matrix), 1)), 0)
    return matrix / matrix.shape[0] ** 0.5


def load_key_shift(num_layers: int, num_kv_heads: int, head_dim: int, device, dtype, *,
                   rotation: torch.Tensor | None = None, tensor_parallel_size: int = 1,
                   tensor_parallel_rank: int = 0) -> torch.Tensor | None:
    """The per-(layer, KV head, channel) constant subtracted from post-RoPE K on its way into the
    cache, from the ``NVFP4_KEY_SHIFT`` sidecar; None when unset. A full-model sidecar is sliced
    along KV heads in contiguous rank order; a rank-local one is kept. With a rotation the constant
    becomes ``c R^T``, computed once in float64 and rounded once into ``dtype``. Nothing adds the
    constant back: ``q.mu`` is the same for every key a query sees, so softmax is unchanged."""
    path = os.environ.get(KEY_SHIFT_ENV)
    if not path:
        return None
    if tensor_parallel_size < 1 or not 0 <= tensor_parallel_rank < tensor_parallel_size:
        raise ValueError(
            f"invalid tensor-parallel coordinates: rank={tensor_parallel_rank}, size={tensor_parallel_size}"
        )
    from safetensors.torch import load_file

    tensors = load_file(path)
    if "key_shift" not in tensors:
        raise ValueError(f"{path} has no 'key_shift' tensor, found {sorted(tensors)}")
    shift = tensors["key_shift"]
    expected = (num_layers, num_kv_heads, head_dim)
    global_shape = (num_layers, num_kv_heads * tensor_parallel_size, head_dim)
    if tensor_parallel_size > 1 and tuple(shift.shape) == global_shape:
        start = tensor_parallel_rank * num_kv_heads
        shift = shift[:, start:start + num_kv_heads, :].contiguous()
    if tuple(shift.shape) != expected:
        raise ValueError(
            f"{path} holds a key_shift of {tuple(shift.shape)}, this model "
            f"needs {expected} (rank-local) or {global_shape} (full-model)"
        )
    return active_shift(shift.to(device), rotation, dtype)


def active_shift(shift: torch.Tensor, rotation: torch.Tensor | None, dtype: torch.dtype) -> torch.Tensor:
    """An original-basis mean in the form the write path subtracts: ``c R^T`` under a rotation,
    computed in float64, rounded once into ``dtype`` (src/nvfp4_vllm/runtime.py:117-126)."""
    if rotation is None:
        return shift.to(dtype)
    return torch.matmul(shift.double(), rotation.to(device=shift.device).double().T).to(dtype).contiguous()


class LayerRuntime:
    """The tail buffers, cache views and scratch one model's attention layers share."""

    def __init__(self, *, num_layers: int, num_slots: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 device, query_terms: int = 1, rotation: str = "none", key_scale_mode: str = DEFAULT_SCALE_MODE,
                 value_scale_mode: str = DEFAULT_SCALE_MODE, key_scale_geometry: str = "local",
                 tensor_parallel_size: int = 1, tensor_parallel_rank: int = 0) -> None:
        if query_terms not in (1, 2):
            raise ValueError(f"query_terms must be 1 or 2, got {query_terms!r}")
        if rotation not in ("none", "hadamard", "block_hadamard_64"):
            raise ValueError(f"rotation must be 'none', 'hadamard', or 'block_hadamard_64', got {rotation!r}")
        if rotation == "block_hadamard_64":
            raise NotImplementedError("rotation='block_hadamard_64' (an unfused BF16 GEMM arm) is not built")
        if key_scale_geometry not in ("local", "gaussian_global"):
            raise ValueError(f"key_scale_geometry must be 'local' or 'gaussian_global', got {key_scale_geometry!r}")
        device = torch.device(device)
        self.num_layers, self.num_kv_heads, self.head_dim = num_layers, num_kv_heads, head_dim
        self.query_terms, self.rotation_name = query_terms, rotation
        self.key_scale_mode, self.value_scale_mode = key_scale_mode, value_scale_mode
        self.key_scale_geometry = key_scale_geometry
        self.fused_rotation = rotation == "hadamard"
        self.rotation = sylvester_hadamard(head_dim, device, torch.float32) if self.fused_rotation else None
        self.key_shift_enabled = True
        # zeroed: attention reads whole tail pages and masks by weight, so rows past a sequence's
        # length must be finite
        shape = (num_layers, num_slots, TAIL_BUFFER_TOKENS, num_kv_heads, head_dim)
        self.tail_key = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.tail_value = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        # the same storage as one run of tokens, which promotion quantizes out of
        self.tail_key_tokens = self.tail_key.view(-1, num_kv_heads, head_dim)
        self.tail_value_tokens = self.tail_value.view(-1, num_kv_heads, head_dim)
        self.key_shift = load_key_shift(
            num_layers, num_kv_heads, head_dim, device, self.key_shift_dtype, rotation=self.rotation,
            tensor_parallel_size=tensor_parallel_size, tensor_parallel_rank=tensor_parallel_rank)
        # FP64 per-(layer, head, channel) sums of the keys seen while a key-smoothing measurement runs
        self.key_shift_sum: torch.Tensor | None = None
        self.key_shift_tokens = 0
        # query scratch, zeroed once (the quantizer rewrites only part of the padded query and of
        # the scale tiles) and shared by every layer
        self.query_padded = torch.zeros(num_slots, RESIDUAL_ROW_TILE, num_heads, head_dim, dtype=torch.bfloat16,
                                        device=device)
        self.query_fp4 = torch.zeros(num_slots, 1, num_heads, head_dim // 2, dtype=torch.uint8, device=device)
        self.query_scales = torch.zeros(num_slots, 1, num_heads, head_dim // (4 * sf_vec_size(key_scale_mode)),
                                        32, 4, 4, dtype=torch.uint8, device=device)
        self.query_fp4_second = torch.zeros_like(self.query_fp4) if query_terms == 2 else None
        self.query_scales_second = torch.zeros_like(self.query_scales) if query_terms == 2 else None
        # split-KV partials for the widest split launch any decode batch of this engine asks for
        from .builder import decode_num_splits

        sms = torch.cuda.get_device_properties(device).multi_processor_count if device.type == "cuda" else 0
        split_rows = max(
            (rows * split_partial_count(rows, num_kv_heads, splits, residual=True, sms=sms)
             for rows in range(1, num_slots + 1)
             if (splits := decode_num_splits(rows, num_kv_heads, sms)) > 1),
            default=0,
        )
        self.split_partial = (torch.empty(split_rows * num_heads * head_dim, dtype=torch.float32, device=device)
                              if split_rows else None)
        self.split_lse = (torch.empty(split_rows * num_heads, dtype=torch.float32, device=device)
                          if split_rows else None)
        self._views: dict[int, tuple] = {}
        self._by_layer: dict[int, tuple] = {}
        self._bases: torch.Tensor | None = None
        self._expected_layer = 0
        self._writer: KVCacheWriter | None = None
        self._writer_shift = None
        self._bound: dict[int, tuple] = {}
        self._promotion: tuple | None = None
        self._promotion_bases = None

    @property
    def key_shift_dtype(self) -> torch.dtype:
        """FP32 where the writers rotate in FP32, else the cache dtype."""
        return torch.float32 if self.fused_rotation else self.tail_key.dtype

    @property
    def query_rotation(self) -> str:
        return "hadamard" if self.fused_rotation else "none"

    @property
    def active_key_shift(self) -> torch.Tensor | None:
        return self.key_shift if self.key_shift_enabled else None

    def set_key_shift_enabled(self, enabled: bool) -> None:
        """Only between requests: keys already cached were stored under the previous setting."""
        if enabled and self.key_shift is None:
            raise ValueError("no shift has been loaded or measured, so there is nothing to enable")
        self.key_shift_enabled = enabled

    def begin_key_shift_measurement(self) -> None:
        """Measure the mean of K instead of removing it, until ``finish_key_shift_measurement``.
        A shift in force is dropped first: measured against a shifted K the result would be the
        residual mean, close to zero (src/nvfp4_vllm/runtime.py:485-501)."""
        self.key_shift = None
        self.key_shift_sum = torch.zeros(self.num_layers, self.num_kv_heads, self.head_dim, dtype=torch.float64,
                                         device=self.tail_key.device)
        self.key_shift_tokens = 0

    def measure_keys(self, layer_index: int, key: torch.Tensor, tokens: int) -> None:
        """Add this step's post-RoPE keys ``key[:tokens]`` of one layer to the running FP64 sums
        (what src/nvfp4_vllm/impl.py:209-216 does with ``key.double().sum``); layer 0 counts the
        tokens for the model, because every layer sees the same ones."""
        if self.key_shift_sum is None or tokens <= 0:
            return
        import bdfp4

        rows = key[:tokens].view(tokens, self.num_kv_heads, self.head_dim)
        bdfp4.key_channel_sums(rows, self.key_shift_sum[layer_index], bdfp4.current_stream(rows.device))
        if layer_index == 0:
            self.key_shift_tokens += tokens

    def finish_key_shift_measurement(self) -> torch.Tensor:
        """Freeze the measured mean and start subtracting it. Returns the mean rounded once into the
        cache dtype, in the original basis (the sidecar's contract); the active value is the same
        mean rotated in float64 and rounded once into ``key_shift_dtype``
        (src/nvfp4_vllm/runtime.py:503-527)."""
        if self.key_shift_sum is None or self.key_shift_tokens == 0:
            raise ValueError(
                "no tokens were measured, so there is no mean to subtract; "
                "begin_key_shift_measurement must precede a forward pass"
            )
        mean = self.key_shift_sum / self.key_shift_tokens
        measured = mean.to(self.tail_key.dtype)
        self.key_shift = active_shift(measured if self.rotation is None else mean, self.rotation,
                                      self.key_shift_dtype)
        self.key_shift_enabled = True
        self.key_shift_sum = None
        self.key_shift_tokens = 0
        return measured

    def transform_query(self, query: torch.Tensor) -> torch.Tensor:
        """The part of Q's basis change the quantizer does not do itself: none in this build."""
        return query

    def key_write(self, layer_index: int, key: torch.Tensor):
        """(K to hand the writers, whether they rotate it, the layer's shift or None)."""
        shift = self.active_key_shift
        return key, self.fused_rotation, None if shift is None else shift[layer_index]

    @property
    def decode_writes_tail(self) -> bool:
        """Whether the decode prefix's query quantizer writes its own tail tokens: whenever the
        shift (if any) is FP32, which is what the fused tail write takes."""
        shift = self.active_key_shift
        return shift is None or shift.dtype == torch.float32

    def views(self, layer_index: int, kv_cache: torch.Tensor) -> tuple:
        """The four NVFP4 regions of one layer's block array (cached by address); also records the
        layer's cache for the promotion base table."""
        key = kv_cache.data_ptr()
        carved = self._views.get(key)
        if carved is None:
            carved = layout.carve(kv_cache, self.num_kv_heads, self.head_dim, self.key_scale_mode)
            self._views[key] = carved
        if self._by_layer.get(layer_index) is not carved:
            self._by_layer[layer_index] = carved
            self._bases = None
        return carved

    def _current_writer(self, carved) -> KVCacheWriter:
        shift = self.active_key_shift
        if self._writer is not None and shift is self._writer_shift:
            return self._writer
        self._writer = KVCacheWriter(
            regions=carved if carved is not None else self._by_layer[min(self._by_layer)],
            key_scale_mode=self.key_scale_mode, value_scale_mode=self.value_scale_mode,
            key_scale_geometry=self.key_scale_geometry, rotate_key=self.fused_rotation, key_shift=shift,
            tail_key=self.tail_key, tail_value=self.tail_value, sink_tokens=SINK_TOKENS)
        self._writer_shift = shift
        return self._writer

    def writer_for(self, layer_index: int, kv_cache: torch.Tensor):
        """The write path's writer and this layer's bound regions; rebuilt when the shift in force
        changes, regions bound once per carved cache."""
        bound = self._bound.get(layer_index)
        if bound is None or bound[0] is not kv_cache:
            carved = self.views(layer_index, kv_cache)
            bound = (kv_cache, self._current_writer(carved).bind_regions(*carved))
            self._bound[layer_index] = bound
        return self._current_writer(None), bound[1]

    @property
    def destination_bases(self) -> torch.Tensor:
        """``[4, num_layers]`` int64: where each layer's four regions start."""
        if self._bases is None:
            missing = [i for i in range(self.num_layers) if i not in self._by_layer]
            if missing:
                raise ValueError(
                    f"layers {missing} have not written their KV cache, so "
                    "promotion has no address to send their pages to"
                )
            self._bases = torch.tensor(
                [[self._by_layer[layer][region].data_ptr() for layer in range(self.num_layers)]
                 for region in range(4)], dtype=torch.int64, device=self.tail_key.device)
        return self._bases

    def promotion_writer(self):
        """The per-layer writer that seals filled tail pages of every layer at once: page roles
        only, no rotation or shift (the tail already holds K in the cache's basis)."""
        bases = self.destination_bases
        if self._promotion is not None and bases is self._promotion_bases:
            return self._promotion
        regions = self._by_layer[0]
        writer = KVCacheWriter(regions=regions, key_scale_mode=self.key_scale_mode,
                               value_scale_mode=self.value_scale_mode,
                               key_scale_geometry=self.key_scale_geometry, destination_bases=bases)
        self._promotion = (writer, writer.bind_regions(*regions))
        self._promotion_bases = bases
        return self._promotion

    def attend_decode_rows(self, layer_index: int, rows: int, *, query, key, value, kv_cache, step, out,
                           softmax_scale: float, query_scale_mode: str) -> None:
        """Decode attention of the batch's first ``rows`` rows (vLLM sorts the one-token rows to the
        front) over this layer's FP4 pages, BF16 tail and sink, written into ``out[:rows]``.

        Everything the kernel call needs that lives here goes in from here: the carved cache, the
        tail buffers, the query and split scratch (so the call allocates nothing), and this layer's
        share of the key transform for the fused tail write. ``step`` is this step's
        ``NVFP4Metadata``; its per-row tensors were written on the device by the control kernel this
        same step, which is why they are passed as trusted: checking them would mean reading them."""
        from nvfp4_decode_kernel import DecodeTailWrite, fp4_decode

        regions = self.views(layer_index, kv_cache)
        per_row = {name: getattr(step, name)[:rows]
                   for name in ("row_to_slot", "seq_lens", "seqused_fp4", "seqused_residual", "seqused_sink")}
        tail_key, tail_value = self.tail_key[layer_index], self.tail_value[layer_index]
        new_token = None
        if self.decode_writes_tail:
            raw_key, rotate, shift = self.key_write(layer_index, key)
            new_token = DecodeTailWrite(
                key=raw_key[:rows], value=value[:rows], tail_key=tail_key, tail_value=tail_value,
                row_to_slot=per_row["row_to_slot"], seq_lens=per_row["seq_lens"], seqused_fp4=per_row["seqused_fp4"],
                rotate_key=rotate, key_shift=shift, sink_tokens=SINK_TOKENS)
        fp4_decode(
            self.transform_query(query[:rows]), *regions, step.block_table[:rows, :step.decode_page_columns],
            per_row["seqused_fp4"],
            residual_key_pages_bf16=tail_key, residual_value_pages_bf16=tail_value,
            residual_page_ids=per_row["row_to_slot"], seqused_residual=per_row["seqused_residual"],
            seqused_sink=per_row["seqused_sink"] if SINK_TOKENS else None,
            softmax_scale=softmax_scale, out=out[:rows], trusted_metadata=True,
            num_splits=step.decode_num_splits, row_order=step.decode_row_order,
            query_terms=self.query_terms, scale_mode=query_scale_mode, query_rotation=self.query_rotation,
            tail_write=new_token,
            query_padded_scratch=self.query_padded, query_fp4_scratch=self.query_fp4,
            query_scales_scratch=self.query_scales, query_fp4_second_scratch=self.query_fp4_second,
            query_scales_second_scratch=self.query_scales_second,
            split_partial_scratch=self.split_partial, split_lse_scratch=self.split_lse)

    def expect_layer(self, layer_index: int) -> None:
        """Refuse a step whose layers do not run in index order: promotion fires after the highest
        index, which is the last layer only if construction order is execution order. The counter
        resynchronises when it complains."""
        if layer_index != self._expected_layer:
            expected = self._expected_layer
            self._expected_layer = (layer_index + 1) % self.num_layers
            raise ValueError(
                f"layer {layer_index} ran where layer {expected} was expected; "
                "promotion assumes layers run in index order"
            )
        self._expected_layer = (layer_index + 1) % self.num_layers
