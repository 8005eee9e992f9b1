"""The CPU arm that ``bench.py`` times beside the GPU path: one decode step of a slice of the workload.

TEST INFRASTRUCTURE (the ``cpu_baseline`` leg and ``--impl reference`` of ``bench.py`` only).
Two implementations of the same step:

* ``kind = "reference"``: the reference's own CPU model, ``oracle/_ref`` (made by ``make_ref.py`` from
  src/nvfp4_decode_kernel/reference.py of OpenBitSys/BitDecoding-FP4), composed as that file's
  docstrings describe the path: Hadamard + two-term NVFP4 query (``nvfp4_two_term``), keys and
  values round-tripped through the cache's formats up front (``nvfp4_round_trip`` with ``four_six``
  along channels, ``value_token_axis_round_trip`` along tokens), then ``online_softmax_pv`` in the
  kernel's block order with FP4 probabilities and the stale-maximum threshold 8.
* ``kind = "port"``: this repository's restatement (``nvfp4_oracle``), which reads the packed cache
  bytes; used when ``oracle/_ref`` is absent.

A step covers one decode row: ``heads_kv`` KV heads with ``ratio`` query heads each, ``context``
tokens, 128 rolling BF16 tokens and ``sink`` BF16 sink tokens. What is quantized up front (the cache)
is not timed; the step quantizes the query, writes the new token into the tail and attends.
"""

from __future__ import annotations

import importlib
import sys
import time
from pathlib import Path

import torch

REF_DIR = Path(__file__).resolve().parent / "_ref"


def load_reference():
    """The reference's ``reference`` module from ``oracle/_ref``, or None."""
    if not (REF_DIR / "nvfp4_decode_kernel_ref" / "reference.py").exists():
        return None
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    return importlib.import_module("nvfp4_decode_kernel_ref.reference")


def _inputs(context: int, heads_kv: int, ratio: int, seed: int):
    gen = torch.Generator().manual_seed(seed)
    k = torch.randn(context, heads_kv, 128, generator=gen)
    for h in range(heads_kv):
        k[:, h, torch.randperm(128, generator=gen)[:4]] *= torch.exp(1.5 * torch.randn(4, generator=gen))
    v = torch.randn(context, heads_kv, 128, generator=gen).to(torch.bfloat16)
    q = torch.randn(heads_kv * ratio, 128, generator=gen).to(torch.bfloat16)
    return k.to(torch.bfloat16), v, q


def reference_step_seconds(ref, context: int, *, heads_kv: int = 1, ratio: int = 4, sink: int = 4, seed: int = 0,
                           repeats: int = 1) -> float:
    """Seconds per decode step of one row on the reference's CPU model."""
    k, v, q = _inputs(context, heads_kv, ratio, seed)
    fp4_tokens = ((context - 1) // 128) * 128
    sink = min(sink, context)
    basis = ref.hadamard_rotate(k).to(torch.bfloat16)            # the cache basis of K, rounded once
    k_cache = ref.nvfp4_round_trip(basis[:fp4_tokens], scale_mode="four_six")
    v_cache = ref.value_token_axis_round_trip(v, fp4_tokens=fp4_tokens, sink_tokens=sink, scale_mode="amax6")
    heads = heads_kv * ratio
    kv_of = torch.arange(heads) // ratio
    start = time.perf_counter()
    for _ in range(repeats):
        rotated = ref.hadamard_rotate(q)
        first, second = ref.nvfp4_two_term(rotated, scale_mode="amax6")
        basis[-1] = ref.hadamard_rotate(k[-1:]).to(torch.bfloat16)[0]  # this step's token into the tail
        scores = torch.empty(heads, context)
        bf16_query = rotated.to(torch.bfloat16).float()
        for h in range(heads):
            kv = int(kv_of[h])
            scores[h, :fp4_tokens] = k_cache[:, kv] @ (first[h] + second[h])
            scores[h, fp4_tokens:] = basis[fp4_tokens:, kv].float() @ bf16_query[h]
            scores[h, :sink] = basis[:sink, kv].float() @ bf16_query[h]
        ref.online_softmax_pv(scores, v_cache[:, kv_of], fp4_tokens=fp4_tokens, quantize_probabilities=True,
                              sink_tokens=sink, softmax_scale=128 ** -0.5, rescale_threshold=8.0)
    return (time.perf_counter() - start) / repeats


def port_step_seconds(context: int, *, heads_kv: int = 1, ratio: int = 4, sink: int = 4, seed: int = 0,
                      repeats: int = 1, page_tokens: int = 64) -> float:
    """Seconds per decode step of one row on this repository's restatement (packed cache bytes)."""
    from . import nvfp4_oracle as oracle

    k, v, q = _inputs(context, heads_kv, ratio, seed)
    fp4 = ((context - 1) // 128) * 128
    sink, tail = min(sink, context), context - fp4
    pages = fp4 // page_tokens
    kc, ks = oracle.quantize_key_pages(k[:fp4].reshape(pages, page_tokens, heads_kv, 128), "four_six", rotate=True)
    vc, vs = oracle.quantize_value_pages(v[:fp4].reshape(pages, page_tokens, heads_kv, 128), "amax6")
    tail_k = torch.zeros(1, 144, heads_kv, 128, dtype=torch.bfloat16)
    tail_v = torch.zeros_like(tail_k)
    basis = oracle.key_cache_basis(k, rotate=True, shift=None)
    tail_k[0, :tail], tail_v[0, :tail] = basis[fp4:], v[fp4:]
    tail_k[0, 128:128 + sink], tail_v[0, 128:128 + sink] = basis[:sink], v[:sink]
    meta = dict(
        page_table=torch.arange(max(pages, 1), dtype=torch.int32)[None], seqused_fp4=torch.tensor([fp4], dtype=torch.int32),
        tail_key=tail_k, tail_value=tail_v, tail_slot_ids=torch.zeros(1, dtype=torch.int32),
        seqused_residual=torch.tensor([tail], dtype=torch.int32), seqused_sink=torch.tensor([sink], dtype=torch.int32))
    start = time.perf_counter()
    for _ in range(repeats):
        qq = oracle.quantize_query(q[None], heads_kv, scale_mode="amax6", terms=2, rotate=True)
        tail_k[0, tail - 1] = oracle.key_cache_basis(k[-1:], rotate=True, shift=None)[0]
        tail_v[0, tail - 1] = v[-1]
        oracle.decode_reference(query_values=qq["values"], query_padded=qq["padded"], key_codes=kc, key_scales=ks,
                                value_codes=vc, value_scales=vs, heads_kv=heads_kv, softmax_scale=128 ** -0.5, **meta)
    return (time.perf_counter() - start) / repeats


def step_seconds(context: int, **options) -> tuple[float, str]:
    """(seconds per step, kind): the reference itself when ``oracle/_ref`` is there, else the port."""
    ref = load_reference()
    if ref is not None:
        options.pop("page_tokens", None)
        return reference_step_seconds(ref, context, **options), "reference"
    return port_step_seconds(context, **options), "port"
