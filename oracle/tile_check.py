"""Parity of a large decode against the CPU oracle on sampled (row, KV head) tiles.

TEST INFRASTRUCTURE ONLY (used by ``tests/`` and by ``bench.py --verify``, after and outside its
timed regions). A full-size decode (tens of thousands of tokens per row, gigabytes of cache) is
far too much for the CPU oracle as a whole, but every (row, KV head) pair is an independent unit
of the decode (src/nvfp4_decode_kernel/fp4_decode_kernel.py:3057 of OpenBitSys/BitDecoding-FP4:
one tile = (row, head[, split])), so the oracle walks a handful of them over exactly the bytes the
kernel read: the row's pages are gathered from the device cache through its page table.
"""

from __future__ import annotations

import torch

from . import mxfp4_oracle
from . import nvfp4_oracle as oracle


def _tile_cache(w, row: int, kv_head: int):
    """One head of the row's pages, in page-table order, as CPU tensors in the oracle's layouts."""
    h, pt = w.heads_kv, w.page_tokens
    pages = int(w.seqused_fp4[row]) // pt
    ids = w.page_table[row, :pages].long()
    blocks = w.blocks[ids].cpu()  # [pages, block bytes]
    mx = getattr(w, "scale_format", "nvfp4") == "mxfp4"
    codes, scales = pt * 64 * h, (pt * 4 * h if mx else pt * 8 * h)  # bytes of one code / scale region
    head_scales = scales // h
    # the NVFP4 scale region is reserved at full size in the block even when MXFP4 uses half of it
    reserved = pt * 8 * h
    if pt == 128:
        key_codes = blocks[:, :codes].reshape(pages, pt, h, 64)[:, :, kv_head:kv_head + 1]
    else:
        key_codes = blocks[:, :codes].reshape(pages, h, pt, 64).permute(0, 2, 1, 3)[:, :, kv_head:kv_head + 1]
    key_scales = blocks[:, codes:codes + scales].reshape(pages, h, head_scales)[:, kv_head:kv_head + 1]
    value_codes = blocks[:, codes + reserved:2 * codes + reserved].reshape(pages, h, 128, pt // 2)[:, kv_head:kv_head + 1]
    value_scales = blocks[:, 2 * codes + reserved:2 * codes + reserved + scales].reshape(pages, h, head_scales)[
        :, kv_head:kv_head + 1]
    return dict(key_codes=key_codes.contiguous(), key_scales=key_scales.contiguous(),
                value_codes=value_codes.contiguous(), value_scales=value_scales.contiguous())


def oracle_tile(w, row: int, kv_head: int, *, terms: int, scale_mode: str, rotate: bool,
                p_mode: str = "amax2_or_amax6_c8", tau: float = oracle.DEFAULT_P_TAU, num_splits: int = 1,
                bf16_split: bool = False, bf16_page_cost: int = 0, with_tail: bool = True, query=None,
                tensor_scales=(1.0, 1.0, 1.0)):
    """BF16 ``[G, 128]``: what the decode must return for the query heads of ``kv_head`` of ``row``.
    ``w`` is a ``bdfp4.workload.Workload`` on the GPU; ``query`` overrides ``w.query``."""
    ratio = w.heads_q // w.heads_kv
    heads = slice(kv_head * ratio, (kv_head + 1) * ratio)
    q_row = (w.query if query is None else query)[row:row + 1, heads].cpu()
    mx = scale_mode.startswith("mxfp4")
    if mx:
        q = mxfp4_oracle.quantize_query(q_row, 1, rule=scale_mode[len("mxfp4_"):], terms=terms, rotate=rotate,
                                        tensor_scale=tensor_scales[1])
    else:
        q = oracle.quantize_query(q_row, 1, scale_mode=scale_mode, terms=terms, rotate=rotate,
                                  tensor_scale=tensor_scales[1])
    cache = _tile_cache(w, row, kv_head)
    pages = cache["key_codes"].shape[0]
    kwargs = {}
    if with_tail:
        slot = int(w.slot_ids[row])
        kwargs = dict(
            tail_key=w.tail_key[0, slot:slot + 1, :, kv_head:kv_head + 1].cpu(),
            tail_value=w.tail_value[0, slot:slot + 1, :, kv_head:kv_head + 1].cpu(),
            tail_slot_ids=torch.zeros(1, dtype=torch.int32), seqused_residual=w.seqused_residual[row:row + 1].cpu(),
            seqused_sink=w.seqused_sink[row:row + 1].cpu() if w.sink_tokens else None)
    reference = mxfp4_oracle.decode_reference if mx else oracle.decode_reference
    extra = {} if mx else dict(p_mode=p_mode, tau=tau)
    out, _, _ = reference(
        query_values=q["values"], query_padded=q["padded"], **cache,
        page_table=torch.arange(max(pages, 1), dtype=torch.int32)[None], seqused_fp4=w.seqused_fp4[row:row + 1].cpu(),
        heads_kv=1, softmax_scale=128 ** -0.5, num_splits=num_splits, bf16_split=bf16_split,
        bf16_page_cost=bf16_page_cost, tensor_scales=tensor_scales, **extra, **kwargs)
    return out[0]


def check_tiles(w, out: torch.Tensor, tiles, **decode_options) -> dict:
    """Compare ``out`` ``[rows, Hq, 128]`` (device) with the oracle on ``tiles`` = [(row, kv_head), ...];
    ``row_splits`` (a list with one part count per row) replaces ``num_splits`` row by row.
    Returns the worst absolute error and the mean relative error over the sampled tiles, in BF16."""
    ratio = w.heads_q // w.heads_kv
    errors, magnitudes, worst, identical, total = [], [], 0.0, 0, 0
    row_splits = decode_options.pop("row_splits", None)  # per-row part counts (a list), if the launch used them
    for row, kv_head in tiles:
        if row_splits is not None:
            decode_options["num_splits"] = int(row_splits[row])
        want = oracle_tile(w, row, kv_head, **decode_options).float()
        got = out[row, kv_head * ratio:(kv_head + 1) * ratio].float().cpu()
        if not torch.isfinite(got).all():
            return {"tiles": len(tiles), "max_abs": float("inf"), "mean_rel": float("inf")}
        err = (got - want).abs()
        worst = max(worst, float(err.max()))
        errors.append(err.mean())
        magnitudes.append(want.abs().mean())
        identical += int((err == 0).sum())
        total += err.numel()
    mean_abs = float(torch.stack(magnitudes).mean())
    mean_rel = float(torch.stack(errors).mean() / max(mean_abs, 1e-12))
    # mean_abs_output and identical say what kind of agreement it was: where one token takes nearly all
    # of a row's probability the output is that token's dequantized V and agreement is exact
    return {"tiles": len(tiles), "max_abs": worst, "mean_rel": mean_rel, "mean_abs_output": mean_abs,
            "identical": f"{identical}/{total}"}
