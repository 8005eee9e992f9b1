"""Seeded synthetic decode workloads: a paged NVFP4 KV cache filled through the writer kernels.

Stands in for real model activations with the distributions the benchmark configuration names:
K, V and Q are BF16 draws from N(0,1); each KV head of K has four outlier channels (fixed for the
whole run) scaled by a lognormal(0, 1.5) factor; the block table is a random permutation of the
physical blocks, with block 0 left unused as the serving engine's null block. The cache uses the
serving engine's block layout: one flat ``[blocks, 2*128*H*72]`` byte tensor whose four regions
(K codes, K scales, V codes, V scales) are strided views
(src/nvfp4_vllm/layout.py:87-130 of OpenBitSys/BitDecoding-FP4).

A sequence of ``n`` tokens holds ``fp4 = ((n-1)//128)*128`` tokens in FP4 pages, the remaining
``n - fp4`` (1..128) in its BF16 rolling tail and its first ``min(n, sink)`` tokens again in the
BF16 sink (src/nvfp4_vllm/control.py:62-89). With ``page_tokens=64`` (no reference counterpart)
the cache is built from 64-token pages, two page-table entries per 128-token step.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

PAGE = 128
HEAD_DIM = 128


def carve_cache(blocks: torch.Tensor, heads: int, page_tokens: int = PAGE, scale_format: str = "nvfp4"):
    """Four region views of a flat ``[num_blocks, 2*page_tokens*H*72]`` u8 cache: K codes, K scales,
    V codes, V scales at byte offsets 0, 64, 72 and 136 times ``page_tokens * H``. An MXFP4 cache
    (128-token pages) keeps those offsets and uses the first half of each scale region."""
    num_blocks, block_bytes = blocks.shape
    assert page_tokens in (128, 64) and block_bytes == 2 * page_tokens * heads * 72
    assert scale_format == "nvfp4" or page_tokens == PAGE
    pitch = blocks.stride(0)
    base, origin = blocks, blocks.storage_offset()
    codes, scales = page_tokens * 64 * heads, page_tokens * 8 * heads  # bytes of one region
    # 128-token pages are token-major [tok][H][64]; a 64-token page is head-major [H][tok][64]
    key_strides = (pitch, heads * 64, 64, 1) if page_tokens == PAGE else (pitch, 64, page_tokens * 64, 1)
    key_codes = base.as_strided((num_blocks, page_tokens, heads, 64), key_strides, origin)
    value_codes = base.as_strided(
        (num_blocks, heads, HEAD_DIM, page_tokens // 2), (pitch, HEAD_DIM * page_tokens // 2, page_tokens // 2, 1),
        origin + codes + scales,
    )
    if page_tokens == PAGE:
        atoms = 1 if scale_format == "mxfp4" else 2
        shape, strides = (num_blocks, 32, 4, 1, 4, atoms, heads), (pitch, 16, 4, atoms * 512, 1, 512, atoms * 512)
        key_scales = base.as_strided(shape, strides, origin + codes)
        value_scales = base.as_strided(shape, strides, origin + 2 * codes + scales)
    else:
        key_scales = base.as_strided((num_blocks, 32, 2, 1, 4, 2, heads), (pitch, 8, 4, 512, 1, 256, 512),
                                     origin + codes)
        value_scales = base.as_strided((num_blocks, 32, 4, 1, 4, 1, heads), (pitch, 16, 4, 512, 1, 512, 512),
                                       origin + 2 * codes + scales)
    return key_codes, key_scales, value_codes, value_scales


def split_lengths(seq_len: int, sink_tokens: int):
    sink = min(seq_len, sink_tokens)
    fp4 = ((seq_len - 1) // PAGE) * PAGE if seq_len else 0
    return sink, fp4, seq_len - fp4


@dataclass
class Workload:
    rows: int
    heads_q: int
    heads_kv: int
    seq_lens: list
    sink_tokens: int
    device: torch.device
    blocks: torch.Tensor = None
    regions: tuple = None
    page_table: torch.Tensor = None
    seqused_fp4: torch.Tensor = None
    seqused_residual: torch.Tensor = None
    seqused_sink: torch.Tensor = None
    tail_key: torch.Tensor = None      # [1, slots, 128+sink, H, 128]
    tail_value: torch.Tensor = None
    slot_ids: torch.Tensor = None
    query: torch.Tensor = None
    key_shift: torch.Tensor | None = None
    rotate: bool = False
    page_tokens: int = PAGE
    scale_format: str = "nvfp4"
    tensor_scales: tuple = (1.0, 1.0, 1.0)  # key, query, value
    outlier_scale: torch.Tensor = None  # [H, 128] multiplicative factors applied to K
    kept: dict = field(default_factory=dict)  # raw BF16 K/V of each row when keep_source

    def algorithmic_bytes(self) -> int:
        """Bytes one decode step must move: FP4 K/V codes and scales, BF16 tail and sink rows,
        query in, output out, and the page-table entries consumed."""
        total = 0
        for n in self.seq_lens:
            sink, fp4, tail = split_lengths(n, self.sink_tokens)
            total += fp4 * self.heads_kv * 144 + (tail + sink) * self.heads_kv * 512 + (fp4 // self.page_tokens) * 4
        return total + self.rows * self.heads_q * HEAD_DIM * 2 * 2


def build_workload(
    *, rows: int, heads_q: int, heads_kv: int, seq_lens, sink_tokens: int = 16, seed: int = 0,
    device="cuda", key_scale_mode: str = "amax6", value_scale_mode: str = "amax6", rotate: bool = False,
    key_shift: bool = False, shuffle: bool = True, keep_source: bool = False, chunk_pages: int = 256,
    page_tokens: int = PAGE, key_tensor_scale: float = 1.0, value_tensor_scale: float = 1.0,
    loud_prefix: int = 0, loud_factor: float = 6.0,
) -> Workload:
    """Generate K/V, quantize them into a paged cache with ``KVCacheWriter`` and fill the BF16
    tail and sink, sequence by sequence so that temporaries stay bounded. An ``mxfp4_*`` key scale mode
    builds an MXFP4 cache. ``loud_prefix`` multiplies the keys of every sequence's first tokens by
    ``loud_factor``: the oldest pages and the sink, which the decode reaches last, then score far
    above what came before them, so the running maximum has to move late in the walk."""
    from nvfp4_decode_kernel.quantize_kv_kernel import KVCacheWriter
    from nvfp4_decode_kernel.scale_mode import scale_format as format_of

    device = torch.device(device)
    seq_lens = [int(n) for n in seq_lens]
    assert len(seq_lens) == rows
    gen = torch.Generator(device=device).manual_seed(seed)
    w = Workload(rows, heads_q, heads_kv, seq_lens, sink_tokens, device, rotate=rotate, page_tokens=page_tokens,
                 scale_format=format_of(key_scale_mode),
                 tensor_scales=(float(key_tensor_scale), 1.0, float(value_tensor_scale)))
    pages_per_row = [split_lengths(n, sink_tokens)[1] // page_tokens for n in seq_lens]
    max_pages = max(1, max(pages_per_row))
    num_blocks = 1 + sum(pages_per_row)
    w.blocks = torch.zeros(num_blocks, 2 * page_tokens * heads_kv * 72, dtype=torch.uint8, device=device)
    w.regions = carve_cache(w.blocks, heads_kv, page_tokens, w.scale_format)
    # the block order has a generator of its own, so the token values do not depend on the page size
    order_gen = torch.Generator(device=device).manual_seed(seed + 0x5EED)
    order = torch.randperm(num_blocks - 1, generator=order_gen, device=device) + 1 if shuffle else torch.arange(
        1, num_blocks, device=device)
    w.page_table = torch.zeros(rows, max_pages, dtype=torch.int32, device=device)
    tail_rows = PAGE + sink_tokens
    w.tail_key = torch.zeros(1, rows, tail_rows, heads_kv, HEAD_DIM, dtype=torch.bfloat16, device=device)
    w.tail_value = torch.zeros_like(w.tail_key)
    w.slot_ids = torch.arange(rows, dtype=torch.int32, device=device)
    # outlier channels: 4 per KV head, fixed for the run
    w.outlier_scale = torch.ones(heads_kv, HEAD_DIM, device=device)
    for h in range(heads_kv):
        channels = torch.randperm(HEAD_DIM, generator=gen, device=device)[:4]
        w.outlier_scale[h, channels] = torch.exp(1.5 * torch.randn(4, generator=gen, device=device))
    if key_shift:
        w.key_shift = (0.25 * torch.randn(1, heads_kv, HEAD_DIM, generator=gen, device=device)).float()
    writer = KVCacheWriter(
        regions=w.regions, key_scale_mode=key_scale_mode, value_scale_mode=value_scale_mode,
        rotate_key=rotate, key_shift=w.key_shift, tail_key=w.tail_key, tail_value=w.tail_value,
        sink_tokens=sink_tokens, key_tensor_scale=key_tensor_scale, value_tensor_scale=value_tensor_scale,
    )
    cursor = 0
    fp4_list, tail_list, sink_list = [], [], []
    for row, n in enumerate(seq_lens):
        sink, fp4, tail = split_lengths(n, sink_tokens)
        fp4_list.append(fp4)
        tail_list.append(tail)
        sink_list.append(sink)
        pages = fp4 // page_tokens
        ids = order[cursor:cursor + pages].to(torch.int32)
        cursor += pages
        w.page_table[row, :pages] = ids
        kept_k, kept_v = [], []
        # FP4 pages, in chunks; the chunk that holds the sequence's last tokens also writes the tail
        starts = list(range(0, fp4, chunk_pages * PAGE)) or [0]
        for start in starts:
            stop = min(fp4, start + chunk_pages * PAGE)
            last = start == starts[-1]
            tokens_here = (n - start) if last else (stop - start)
            k = torch.randn(tokens_here, heads_kv, HEAD_DIM, generator=gen, device=device)
            k = k * w.outlier_scale
            if start < loud_prefix:
                k[:loud_prefix - start] *= loud_factor
            k = k.to(torch.bfloat16)
            v = torch.randn(tokens_here, heads_kv, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
            if keep_source:
                kept_k.append(k)
                kept_v.append(v)
            chunk = (stop - start) // page_tokens
            source_tokens = torch.arange(chunk, dtype=torch.int32, device=device) * page_tokens
            destination = ids[start // page_tokens:start // page_tokens + chunk].contiguous()
            if last or (start == 0 and sink):
                # a one-row "prefill" whose computed prefix is `start`: tail candidates cover the
                # rolling page past the FP4 prefix and the sink positions this chunk holds
                qsl = torch.tensor([0, tokens_here], dtype=torch.int32, device=device)
                seq = torch.tensor([start + tokens_here], dtype=torch.int32, device=device)
                used = torch.tensor([fp4 if last else start + tokens_here], dtype=torch.int32, device=device)
                slot = torch.tensor([row], dtype=torch.int32, device=device)
                writer(k, v, w.regions, source_tokens, destination, qsl, seq, used, slot, 0, 0, 0)
            else:
                empty = torch.zeros(0, dtype=torch.int32, device=device)
                qsl = torch.zeros(1, dtype=torch.int32, device=device)
                writer(k, v, w.regions, source_tokens, destination, qsl, empty, empty, empty, 0, 0, 0)
        if keep_source:
            w.kept[row] = (torch.cat(kept_k), torch.cat(kept_v))
    w.seqused_fp4 = torch.tensor(fp4_list, dtype=torch.int32, device=device)
    w.seqused_residual = torch.tensor(tail_list, dtype=torch.int32, device=device)
    w.seqused_sink = torch.tensor(sink_list, dtype=torch.int32, device=device)
    w.query = torch.randn(rows, heads_q, HEAD_DIM, generator=gen, device=device).to(torch.bfloat16)
    return w
