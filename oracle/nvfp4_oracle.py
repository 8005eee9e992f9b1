"""CPU oracle for the NVFP4 quantize-on-write and paged FP4 decode-attention path.

TEST INFRASTRUCTURE ONLY. Nothing under the product package may import this module; it
is the checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline
leg of ``bench.py``. It restates, in plain PyTorch on the CPU, the algorithm of
OpenBitSys/BitDecoding-FP4; every function cites the file:line of that project it follows.
Parity is pinned: ``tests/golden/make_golden.py`` runs the reference's own
``src/nvfp4_decode_kernel/reference.py`` on seeded inputs and the committed fixtures are
checked against this restatement by ``tests/test_oracle_golden.py``.

Layouts (bytes) follow src/nvfp4_decode_kernel/quantize_kv_kernel.py:115-120,671-675:
  K codes  [page][128 tok][H][64]     byte b of a head vector = channels (2b, 2b+1), low nibble first
  V codes  [page][H][128 ch][64]      byte b = tokens (2b, 2b+1)
  scales   [page][H][2][32][4][4]     (row r, group g) at (g//4)*512 + (r%32)*16 + (r//32)*4 + g%4
"""

from __future__ import annotations

import math

import torch

PAGE = 128
HEAD_DIM = 128
GROUP = 16
SINK_TOKENS = 16
RESCALE_THRESHOLD = 8.0  # src/nvfp4_decode_kernel/fp4_decode_kernel.py:93
DEFAULT_P_TAU = 21.0 / 1024.0  # src/nvfp4_decode_kernel/p_scale.py:14

# src/nvfp4_decode_kernel/scale_mode.py:18-22
SCALE_MODES = {"amax6": (6.0,), "four_six": (6.0, 4.0), "four_six_sixhalf": (6.0, 4.0, 6.5)}
SCALE_MODE_IDS = {"amax6": 0, "four_six": 1, "four_six_sixhalf": 2}

_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=torch.float32)
_E4M3_MAX = 448.0


# --------------------------------------------------------------------------------------
# element conversions
# --------------------------------------------------------------------------------------

def e2m1_index(magnitude: torch.Tensor) -> torch.Tensor:
    """Index 0..7 of the E2M1 magnitude nearest to ``magnitude`` (>= 0), ties to the even
    code, saturating at 6: the behaviour of ``cvt.rn.satfinite.e2m1x2.f32``
    (src/nvfp4_decode_kernel/reference.py:50-79). Written as comparisons against the seven
    midpoints: a tie goes down at an even-indexed midpoint and up at an odd one."""
    m = magnitude
    index = torch.zeros_like(m, dtype=torch.int32)
    midpoints = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
    for k, mid in enumerate(midpoints):
        # boundary k separates codes k and k+1; code k is even when k is even
        step = (m > mid) if k % 2 == 0 else (m >= mid)
        index = index + step.to(torch.int32)
    return index


def e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """Four-bit codes, sign in bit 3 (src/nvfp4_decode_kernel/reference.py:82-95). The sign
    bit follows the sign bit of ``x`` itself, so -0.0 encodes as 8 like any negative value
    that rounds to zero, which is what the hardware conversion emits."""
    x = x.float()
    sign = torch.signbit(x)
    return (e2m1_index(x.abs()) | torch.where(sign, 8, 0)).to(torch.uint8)


def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    codes = codes.to(torch.int64)
    magnitude = _E2M1_VALUES[codes & 7]
    return torch.where((codes & 8) != 0, -magnitude, magnitude)


def e4m3_round(x: torch.Tensor) -> torch.Tensor:
    """Non-negative FP32 -> E4M3 (RN-even, saturating at 448) -> FP32
    (src/nvfp4_decode_kernel/reference.py:30-36,138-140)."""
    return x.float().clamp(max=_E4M3_MAX).to(torch.float8_e4m3fn).float()


def e4m3_bytes(x: torch.Tensor) -> torch.Tensor:
    return x.float().clamp(max=_E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_from_bytes(b: torch.Tensor) -> torch.Tensor:
    return b.contiguous().view(torch.float8_e4m3fn).float()


# --------------------------------------------------------------------------------------
# block-scale search
# --------------------------------------------------------------------------------------

def _fma_squares(difference: torch.Tensor) -> torch.Tensor:
    """sum of squares accumulated with one FP32 rounding per element, in element order
    (src/nvfp4_decode_kernel/_block_scale.py:262-269; float64 emulation argument in
    src/nvfp4_decode_kernel/reference.py:98-125)."""
    total = torch.zeros(difference.shape[:-1], dtype=torch.float32)
    wide = difference.double()
    for i in range(difference.shape[-1]):
        total = (total.double() + wide[..., i] * wide[..., i]).float()
    return total


def quantize_groups(groups: torch.Tensor, scale_mode: str = "amax6"):
    """Quantize ``[..., 16]`` FP32 groups.

    Returns (codes u8 ``[..., 16]``, scale FP32 ``[...]`` holding an E4M3 value, winner int64).
    Follows select_group_scale / _round_trip / _candidate_scale
    (src/nvfp4_decode_kernel/_block_scale.py:218-327) and nvfp4_quantize
    (src/nvfp4_decode_kernel/reference.py:149-204).
    """
    groups = groups.float()
    amax = groups.abs().amax(dim=-1)
    best = None
    for index, divisor in enumerate(SCALE_MODES[scale_mode]):
        reciprocal = torch.tensor(1.0 / divisor, dtype=torch.float32)
        scale = e4m3_round(amax * reciprocal)
        inverse = 1.0 / (scale + torch.tensor(1.0e-30, dtype=torch.float32))
        codes = e2m1_codes(groups * inverse[..., None])
        values = e2m1_decode(codes) * scale[..., None]
        error = _fma_squares(values - groups)
        if best is None:
            best = [codes, scale, error, torch.zeros_like(amax, dtype=torch.int64)]
            continue
        better = error < best[2]
        best[0] = torch.where(better[..., None], codes, best[0])
        best[1] = torch.where(better, scale, best[1])
        best[2] = torch.where(better, error, best[2])
        best[3] = torch.where(better, torch.full_like(best[3], index), best[3])
    return best[0], best[1], best[3]


def quantize_last_axis(x: torch.Tensor, scale_mode: str = "amax6"):
    """Groups of 16 along the last axis. Returns (codes ``x.shape`` u8, scales ``[..., n/16]``)."""
    groups = x.float().reshape(*x.shape[:-1], x.shape[-1] // GROUP, GROUP)
    codes, scale, _ = quantize_groups(groups, scale_mode)
    return codes.reshape(x.shape), scale


def dequantize_last_axis(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    values = e2m1_decode(codes).reshape(*codes.shape[:-1], codes.shape[-1] // GROUP, GROUP)
    return (values * scales[..., None]).reshape(codes.shape)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """``[..., n]`` codes -> ``[..., n/2]`` bytes, even element in the low nibble
    (src/nvfp4_decode_kernel/_block_scale.py:75-117)."""
    c = codes.to(torch.uint8)
    return c[..., 0::2] | (c[..., 1::2] << 4)


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    p = packed.to(torch.uint8)
    out = torch.stack((p & 15, p >> 4), dim=-1)
    return out.reshape(*p.shape[:-1], p.shape[-1] * 2)


# --------------------------------------------------------------------------------------
# Hadamard rotation and the K cache basis
# --------------------------------------------------------------------------------------

def hadamard_rotate(x: torch.Tensor) -> torch.Tensor:
    """Last axis times the normalised Sylvester Hadamard: FP32 butterflies over the index bits,
    lowest first, then one multiply by fl32(1/sqrt(n)) (src/nvfp4_decode_kernel/reference.py:217-239,
    src/nvfp4_decode_kernel/quantize_q_kernel.py:87-135)."""
    n = x.shape[-1]
    values = x.float().clone()
    lead = values.shape[:-1]
    stride = 1
    while stride < n:
        v = values.reshape(*lead, n // (2 * stride), 2, stride)
        lo, hi = v[..., 0, :], v[..., 1, :]
        values = torch.stack((lo + hi, lo - hi), dim=-2).reshape(*lead, n)
        stride *= 2
    return values * torch.tensor(1.0 / math.sqrt(n), dtype=torch.float32)


def key_cache_basis(key: torch.Tensor, *, rotate: bool, shift: torch.Tensor | None) -> torch.Tensor:
    """Raw K ``[..., H, 128]`` BF16 -> the BF16 values the cache stores: rotate, subtract the
    shift ``[H, 128]`` (already in the rotated basis) with a separately rounded subtract, round
    to BF16 once (src/nvfp4_decode_kernel/quantize_kv_kernel.py:123-162)."""
    if not rotate and shift is None:
        return key
    work = hadamard_rotate(key) if rotate else key.float()
    if shift is not None:
        work = work - shift.float()
    return work.to(torch.bfloat16)


# --------------------------------------------------------------------------------------
# page layouts
# --------------------------------------------------------------------------------------

def scale_tile_offsets() -> torch.Tensor:
    """``[128 rows, 8 groups]`` byte offsets inside one head's 1024-byte scale tile."""
    r = torch.arange(128)[:, None]
    g = torch.arange(8)[None, :]
    return (g // 4) * 512 + (r % 32) * 16 + (r // 32) * 4 + (g % 4)


def pack_scale_tile(scales: torch.Tensor) -> torch.Tensor:
    """``[..., rows<=128, 8]`` E4M3-valued FP32 -> ``[..., 1024]`` bytes (unused rows zero)."""
    lead = scales.shape[:-2]
    rows = scales.shape[-2]
    tile = torch.zeros(*lead, 1024, dtype=torch.uint8)
    offsets = scale_tile_offsets()[:rows].reshape(-1)
    tile[..., offsets] = e4m3_bytes(scales).reshape(*lead, rows * 8)
    return tile


def unpack_scale_tile(tile: torch.Tensor, rows: int = 128) -> torch.Tensor:
    offsets = scale_tile_offsets()[:rows].reshape(-1)
    picked = tile[..., offsets]
    return e4m3_from_bytes(picked).reshape(*tile.shape[:-1], rows, 8)


def key_scale_offsets64() -> torch.Tensor:
    """``[64 tokens, 8 groups]`` byte offsets inside one head's 512-byte K scale block of a
    64-token page: two half atoms ``[group // 4][token % 32][token // 32][group % 4]``. The
    reference has no 64-token page (src/nvfp4_decode_kernel/_decode.py:23 pins 128); this is the
    CUDA path's own layout, whose values must equal those of the 128-token page."""
    t = torch.arange(64)[:, None]
    g = torch.arange(8)[None, :]
    return (g // 4) * 256 + (t % 32) * 8 + (t // 32) * 4 + (g % 4)


def _place_chunks(packed: torch.Tensor, row_key: torch.Tensor) -> torch.Tensor:
    """Move the 16-byte chunks of each row (last axis) to position ``chunk ^ row_key``; ``row_key``
    broadcasts against ``packed.shape[:-1]``. The move is its own inverse. 64-token pages store
    their code rows this way: the placement of the 64- or 32-byte shared-memory swizzle the decode
    kernel's MMA reads, so that a page is fetched as it lies."""
    chunks = packed.reshape(*packed.shape[:-1], packed.shape[-1] // 16, 16)
    position = torch.arange(chunks.shape[-2]) ^ row_key.expand(packed.shape[:-1])[..., None]
    return torch.gather(chunks, -2, position[..., None].expand_as(chunks)).reshape(packed.shape)


def _key_chunk_key() -> torch.Tensor:
    return ((torch.arange(64) >> 1) & 3)[:, None]  # [tokens, 1] against [pages, tokens, H]


def _value_chunk_key() -> torch.Tensor:
    return (torch.arange(128) >> 2) & 1  # [channels] against [pages, H, channels]


def divide_by_tensor_scale(x: torch.Tensor, tensor_scale: float) -> torch.Tensor:
    """``x / tensor_scale`` as the CUDA path forms it: FP32 values times fl32(1 / tensor_scale), one
    rounding. The reference has no per-tensor scale (src/nvfp4_decode_kernel/_block_scale.py:272-289
    stores the E4M3 block scale alone); 1.0 leaves ``x`` untouched, which is the pinned arithmetic."""
    if tensor_scale == 1.0:
        return x
    inverse = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(tensor_scale, dtype=torch.float32)
    return x.float() * inverse


def quantize_key_pages(key_pages: torch.Tensor, scale_mode: str = "amax6", *, rotate: bool = False,
                       shift: torch.Tensor | None = None, tensor_scale: float = 1.0):
    """``[pages, 128, H, 128]`` BF16 -> (codes u8 ``[pages,128,H,64]``, scales u8 ``[pages,H,1024]``).
    Groups run along channels (src/nvfp4_decode_kernel/quantize_kv_kernel.py:165-221).
    A 64-token page ``[pages, 64, H, 128]`` gives codes ``[pages,64,H,64]`` (chunk j of token t at
    position ``j ^ ((t >> 1) & 3)``; in memory the page is head-major) and scales ``[pages,H,512]``."""
    basis = divide_by_tensor_scale(key_cache_basis(key_pages, rotate=rotate, shift=shift), tensor_scale)
    codes, scales = quantize_last_axis(basis, scale_mode)  # scales [pages,tok,H,8]
    if key_pages.shape[1] == 64:
        by_head = e4m3_bytes(scales).permute(0, 2, 1, 3)  # [pages,H,64,8]
        block = torch.zeros(*by_head.shape[:2], 512, dtype=torch.uint8)
        block[..., key_scale_offsets64().reshape(-1)] = by_head.reshape(*by_head.shape[:2], 512)
        return _place_chunks(pack_nibbles(codes), _key_chunk_key()), block
    return pack_nibbles(codes), pack_scale_tile(scales.permute(0, 2, 1, 3))


def quantize_value_pages(value_pages: torch.Tensor, scale_mode: str = "amax6", *, tensor_scale: float = 1.0):
    """``[pages, 128, H, 128]`` BF16 -> (codes u8 ``[pages,H,128,64]``, scales u8 ``[pages,H,1024]``).
    Groups run along the page's tokens (src/nvfp4_decode_kernel/quantize_kv_kernel.py:224-255,
    src/nvfp4_decode_kernel/reference.py:479-525). A 64-token page gives codes ``[pages,H,128,32]``
    (chunk j of channel c at position ``j ^ ((c >> 2) & 1)``) and scales ``[pages,H,512]``: the
    first atom of the 128-token tile (token groups 0-3)."""
    by_channel = divide_by_tensor_scale(value_pages.permute(0, 2, 3, 1), tensor_scale)  # [pages,H,ch,tok]
    codes, scales = quantize_last_axis(by_channel, scale_mode)  # scales [pages,H,ch,tok/16]
    if value_pages.shape[1] == 64:
        padded = torch.cat([scales, torch.zeros_like(scales)], dim=-1)
        return _place_chunks(pack_nibbles(codes), _value_chunk_key()), pack_scale_tile(padded)[..., :512].contiguous()
    return pack_nibbles(codes), pack_scale_tile(scales)


def dequantize_key_pages(codes: torch.Tensor, scale_tiles: torch.Tensor) -> torch.Tensor:
    """Inverse layout walk: -> FP32 ``[pages, tokens, H, 128]`` (tokens = 128, or 64 from the
    64-token layout, told apart by the code tensor's shape)."""
    if codes.shape[1] == 64:
        codes = _place_chunks(codes, _key_chunk_key())
    nib = unpack_nibbles(codes)  # [pages,tok,H,128]
    if codes.shape[1] == 64:
        picked = scale_tiles[..., key_scale_offsets64().reshape(-1)]
        scales = e4m3_from_bytes(picked).reshape(*scale_tiles.shape[:-1], 64, 8).permute(0, 2, 1, 3)
    else:
        scales = unpack_scale_tile(scale_tiles).permute(0, 2, 1, 3)  # [pages,128,H,8]
    return dequantize_last_axis(nib, scales)


def dequantize_value_pages(codes: torch.Tensor, scale_tiles: torch.Tensor) -> torch.Tensor:
    if codes.shape[-1] == 32:
        codes = _place_chunks(codes, _value_chunk_key())
    nib = unpack_nibbles(codes)  # [pages,H,ch,tok]
    if codes.shape[-1] == 32:
        padded = torch.cat([scale_tiles, torch.zeros_like(scale_tiles)], dim=-1)
        scales = unpack_scale_tile(padded)[..., :4]  # [pages,H,ch,4]
    else:
        scales = unpack_scale_tile(scale_tiles)  # [pages,H,ch,8]
    return dequantize_last_axis(nib, scales).permute(0, 3, 1, 2)


# --------------------------------------------------------------------------------------
# decode query
# --------------------------------------------------------------------------------------

def quantize_query(query: torch.Tensor, heads_kv: int, *, scale_mode: str = "amax6", terms: int = 1,
                   rotate: bool = False, tensor_scale: float = 1.0):
    """``[rows, Hq, 128]`` BF16 -> dict with per-term codes ``[rows,1,Hq,64]`` u8, scale storage
    ``[rows,1,Hq,2,32,4,4]`` u8 (zero where nothing is written), the padded-copy values
    ``[rows,Hq,128]`` BF16, and per-term round-trip values FP32.

    Follows _quantize_query_group / _store_term (src/nvfp4_decode_kernel/quantize_q_kernel.py:276-334,
    431-515) and the storage view of src/nvfp4_decode_kernel/_quantize.py:100-132: head ``h`` writes
    row ``h % G`` of the 1024-byte tile at head slot ``h // G``.
    """
    rows, heads_q, dim = query.shape
    ratio = heads_q // heads_kv
    values = hadamard_rotate(query) if rotate else query.float()
    padded = values.to(torch.bfloat16)  # the BF16 copy is never divided by the tensor scale
    out = {"padded": padded, "codes": [], "scales": [], "values": []}
    current = divide_by_tensor_scale(values, tensor_scale)
    for _ in range(terms):
        codes, scales = quantize_last_axis(current, scale_mode)  # [rows,Hq,128], [rows,Hq,8]
        storage = torch.zeros(rows, heads_q, 1024, dtype=torch.uint8)
        offsets = scale_tile_offsets()  # [128,8]
        scale_bytes = e4m3_bytes(scales)
        for h in range(heads_q):
            storage[:, h // ratio, offsets[h % ratio]] = scale_bytes[:, h]
        recon = dequantize_last_axis(codes, scales)
        out["codes"].append(pack_nibbles(codes).reshape(rows, 1, heads_q, 64))
        out["scales"].append(storage.reshape(rows, 1, heads_q, 2, 32, 4, 4))
        out["values"].append(recon)
        # x - mag*scale with one rounding (src/nvfp4_decode_kernel/_block_scale.py:602-623)
        current = current - recon
    return out


# --------------------------------------------------------------------------------------
# sequence bookkeeping
# --------------------------------------------------------------------------------------

def split_sequence_length(seq_len: int, sink_tokens: int = SINK_TOKENS, page: int = PAGE):
    """(sink, fp4, residual) lengths (src/nvfp4_vllm/control.py:62-89)."""
    sink = min(seq_len, sink_tokens)
    fp4 = ((seq_len - 1) // page) * page if seq_len else 0
    return sink, fp4, seq_len - fp4


# --------------------------------------------------------------------------------------
# softmax-probability operand
# --------------------------------------------------------------------------------------

def probability_quantize(p: torch.Tensor, mode: str = "amax2_or_amax6_c8", tau: float = DEFAULT_P_TAU):
    """P ``[..., n]`` (n % 16 == 0) -> the values the PV MMA sees. The code is taken with the
    unrounded FP32 scale, the multiplier is the E4M3-rounded scale
    (src/nvfp4_decode_kernel/reference.py:386-464; kernel: fp4_decode_kernel.py:5670-5846,
    _fa4/softmax.py:80-112). ``p`` is already multiplied by 8 under the ``_c8`` mode by the caller."""
    groups = p.float().reshape(*p.shape[:-1], p.shape[-1] // GROUP, GROUP)
    amax = groups.abs().amax(dim=-1, keepdim=True)
    if mode in ("amax2_or_amax6", "amax2_or_amax6_c8"):
        low = amax <= torch.tensor(tau, dtype=torch.float32)
        reciprocal = torch.where(low, torch.tensor(0.5), torch.tensor(1.0 / 6.0, dtype=torch.float32))
    elif mode == "amax6":
        reciprocal = torch.tensor(1.0 / 6.0, dtype=torch.float32)
    else:
        raise ValueError(mode)
    raw = amax * reciprocal
    stored = e4m3_round(raw)
    codes = e2m1_codes(groups * (1.0 / (raw + 1.0e-30)))
    return (e2m1_decode(codes) * stored).reshape(p.shape)


# --------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------

def online_attention(blocks, *, softmax_scale: float, p_mode: str = "amax2_or_amax6_c8",
                     tau: float = DEFAULT_P_TAU, rescale_threshold: float = RESCALE_THRESHOLD,
                     p_quantizer=None):
    """Online softmax over ``blocks`` in the order given, for the query heads of one KV head.

    Each block is ``(scores [G, n], values [n, D], kind)``: raw (unscaled) QK products with masked
    positions already at -inf, the block's V rows, and ``"fp4"`` or ``"bf16"`` for how the
    probabilities reach the PV product. Follows the decode kernel's softmax
    (src/nvfp4_decode_kernel/fp4_decode_kernel.py:5352-5854 for FP4 pages, :4830-5055 for the BF16
    tail and sink) and its CPU model (src/nvfp4_decode_kernel/reference.py:528-641):

    * the first block takes its own maximum; afterwards a running maximum that would grow by at
      most ``rescale_threshold`` powers of two is kept and P is formed against the stale one;
    * under a ``_c8`` mode the probabilities are 8*p (the LSE is corrected by -3 ln 2);
    * the denominator sums the unquantised probabilities;
    * FP4 blocks quantise P per 16 positions (:func:`probability_quantize`), BF16 blocks round it
      to BF16.

    ``p_quantizer`` replaces the NVFP4 rule for FP4 blocks (the MXFP4 operand: a callable from the
    probabilities ``[G, n]`` to the values the PV product sees); ``p_mode`` then only decides the
    ``_c8`` shift.

    Returns ``(out [G, D] FP32 normalised, lse [G] natural log)``; a row nothing contributed to
    has out 0 and lse -inf.
    """
    groups = blocks[0][0].shape[0]
    dim = blocks[0][1].shape[-1]
    scale_log2 = torch.tensor(softmax_scale * math.log2(math.e), dtype=torch.float32)
    shift = 3.0 if p_mode.endswith("_c8") else 0.0
    base_mode = p_mode[:-3] if p_mode.endswith("_c8") else p_mode
    out = torch.zeros(groups, dim, dtype=torch.float32)
    row_max = torch.full((groups,), -torch.inf, dtype=torch.float32)
    row_sum = torch.zeros(groups, dtype=torch.float32)

    def finite(m):
        return torch.where(torch.isinf(m) & (m < 0), torch.zeros_like(m), m)

    for index, (block_scores, block_values, kind) in enumerate(blocks):
        block_scores = block_scores.float()
        block_max = block_scores.amax(dim=-1)
        if index == 0:
            new_max = block_max
            acc = torch.zeros(groups)
        else:
            new_max = torch.maximum(row_max, block_max)
            growth = (row_max - finite(new_max)) * scale_log2
            keep = (growth >= -rescale_threshold) if rescale_threshold > 0 else torch.zeros(groups, dtype=torch.bool)
            new_max = torch.where(keep, row_max, new_max)
            acc = torch.where(keep, torch.ones(groups), torch.exp2(growth))
            acc = torch.where(torch.isnan(acc), torch.zeros_like(acc), acc)
        max_scaled = finite(new_max) * scale_log2 - shift
        p = torch.exp2(block_scores * scale_log2 - max_scaled[:, None])
        row_sum = row_sum * acc + p.sum(dim=-1)
        if kind != "fp4":
            used = p.to(torch.bfloat16).float()
        elif p_quantizer is not None:
            used = p_quantizer(p)
        else:
            used = probability_quantize(p, base_mode, tau)
        out = out * acc[:, None] + used @ block_values.float()
        row_max = new_max

    empty = (row_sum == 0) | torch.isnan(row_sum)
    denom = torch.where(empty, torch.ones_like(row_sum), row_sum)
    result = torch.where(empty[:, None], torch.zeros_like(out), out / denom[:, None])
    lse = (finite(row_max) * scale_log2 + torch.log2(denom) - shift) * math.log(2.0)
    lse = torch.where(empty, torch.full_like(lse, -torch.inf), lse)
    return result, lse


def kernel_order_blocks(*, scores_fp4, values_fp4, fp4_tokens: int, scores_tail=None, values_tail=None,
                        tail_tokens: int = 0, scores_sink=None, values_sink=None, sink_tokens: int = 0,
                        page_range=None, with_bf16: bool = True, page: int = PAGE):
    """The block list of one (row, KV head) in the decode kernel's order: BF16 tail, FP4 pages from
    newest to oldest, BF16 sink (src/nvfp4_decode_kernel/reference.py:542-546,614-640).

    Page 0's first ``sink_tokens`` positions are masked because the sink holds them in BF16
    (fp4_decode_kernel.py:5433-5439); while the FP4 prefix is still empty the same positions are
    masked in the tail instead (:4886-4894). A tail or sink block is always a full 128-row tile
    with the rows past its length masked, as the kernel runs it. ``page_range`` = (first, last)
    restricts the pages (split-KV); ``with_bf16`` says whether this part owns the tail and sink.
    A part with no page at all still runs one fully masked FP4 step (:4729-4733).
    """
    blocks = []
    groups = (scores_fp4 if scores_fp4 is not None else scores_tail).shape[0]
    dim = (values_fp4 if values_fp4 is not None else values_tail).shape[-1]
    if with_bf16 and scores_tail is not None:
        padded = torch.full((groups, page), -torch.inf)
        padded[:, :tail_tokens] = scores_tail[:, :tail_tokens].float()
        if fp4_tokens == 0 and sink_tokens:
            padded[:, :sink_tokens] = -torch.inf
        rows = torch.zeros(page, dim)
        rows[:tail_tokens] = values_tail[:tail_tokens].float()
        blocks.append((padded, rows, "bf16"))
    first, last = (0, fp4_tokens // page) if page_range is None else page_range
    for index in range(last - 1, first - 1, -1):
        block_scores = scores_fp4[:, index * page:(index + 1) * page].float().clone()
        if index == 0 and sink_tokens:
            block_scores[:, :sink_tokens] = -torch.inf
        blocks.append((block_scores, values_fp4[index * page:(index + 1) * page], "fp4"))
    if last <= first:
        blocks.append((torch.full((groups, page), -torch.inf), torch.zeros(page, dim), "fp4"))
    if with_bf16 and scores_sink is not None:
        padded = torch.full((groups, page), -torch.inf)
        padded[:, :sink_tokens] = scores_sink[:, :sink_tokens].float()
        rows = torch.zeros(page, dim)
        rows[:sink_tokens] = values_sink[:sink_tokens].float()
        blocks.append((padded, rows, "bf16"))
    return blocks


def split_page_range(pages: int, num_splits: int, split: int, bf16_page_cost: int = 0):
    """Pages ``[first, last)`` of split ``split``: contiguous chunks of ceil(pages/num_splits)
    (src/nvfp4_decode_kernel/_fa4/block_info.py:47-54). ``bf16_page_cost`` (not in the reference;
    the CUDA path's load balance) charges split 0 that many pages for the tail and sink it also
    merges: chunks of ceil((pages + cost)/num_splits), split 0 shortened by the cost."""
    chunk = -(-(pages + bf16_page_cost) // num_splits) if (pages + bf16_page_cost) else 0
    first_chunk = max(chunk - bf16_page_cost, 0)
    if split == 0:
        return 0, min(first_chunk, pages)
    first = min(first_chunk + (split - 1) * chunk, pages)
    return first, min(first + chunk, pages)


def decode_reference(*, query_values, query_padded, key_codes, key_scales, value_codes, value_scales,
                     page_table, seqused_fp4, heads_kv: int, softmax_scale: float,
                     tail_key=None, tail_value=None, tail_slot_ids=None, seqused_residual=None,
                     seqused_sink=None, p_mode: str = "amax2_or_amax6_c8", tau: float = DEFAULT_P_TAU,
                     num_splits: int = 1, bf16_split: bool = False, bf16_page_cost: int = 0,
                     rescale_threshold: float = RESCALE_THRESHOLD, tensor_scales=(1.0, 1.0, 1.0),
                     dequantize_pages=None, p_quantizer=None):
    """Whole-batch decode attention from the packed cache, as the CUDA path is asked to compute it.

    ``query_values`` is a list of one or two FP32 ``[rows, Hq, 128]`` reconstructions of the FP4
    query terms (their QK products are summed, fp4_decode_kernel.py:5418-5420); ``query_padded``
    ``[rows, Hq, 128]`` BF16 scores the tail and the sink. Cache regions are the packed byte
    layouts of this module. Returns ``(out BF16 [rows,Hq,128], partial_out, partial_lse)`` where the
    partials are ``[parts, rows, Hq, 128]`` / ``[parts, rows, Hq]`` FP32 (parts = 1 when unsplit).

    ``tensor_scales`` = (key, query, value) FP32 per-tensor scales (no reference counterpart; parity
    unpinned away from 1.0): FP4-page scores are multiplied by fl32(key * query), FP4-page values by
    the value scale. ``dequantize_pages`` = (key_fn, value_fn) and ``p_quantizer`` swap in another
    scale format (MXFP4, ``oracle/mxfp4_oracle.py``) for the pages and the probability operand.
    """
    rows, heads_q, dim = query_values[0].shape
    ratio = heads_q // heads_kv
    parts = num_splits + (1 if (bf16_split and num_splits > 1) else 0)
    partial_out = torch.zeros(parts, rows, heads_q, dim)
    partial_lse = torch.full((parts, rows, heads_q), -torch.inf)
    has_tail = tail_key is not None
    has_sink = has_tail and seqused_sink is not None
    key_fn, value_fn = dequantize_pages or (dequantize_key_pages, dequantize_value_pages)
    score_scale = torch.tensor(tensor_scales[0], dtype=torch.float32) * torch.tensor(tensor_scales[1], dtype=torch.float32)
    value_scale = torch.tensor(tensor_scales[2], dtype=torch.float32)
    for row in range(rows):
        fp4_tokens = int(seqused_fp4[row])
        pages = fp4_tokens // PAGE  # 128-token steps of the walk, whatever the cache page size
        ids = page_table[row, :fp4_tokens // key_codes.shape[1]].long()
        slot = int(tail_slot_ids[row]) if has_tail else -1
        tail_tokens = int(seqused_residual[row]) if has_tail and slot >= 0 else 0
        sink_tokens = int(seqused_sink[row]) if has_sink and slot >= 0 else 0
        slot = max(slot, 0)
        for kvh in range(heads_kv):
            heads = slice(kvh * ratio, (kvh + 1) * ratio)
            if pages:
                k = key_fn(key_codes[ids][:, :, kvh:kvh + 1], key_scales[ids][:, kvh:kvh + 1])
                v = value_fn(value_codes[ids][:, kvh:kvh + 1], value_scales[ids][:, kvh:kvh + 1])
                k = k.reshape(fp4_tokens, dim)
                v = v.reshape(fp4_tokens, dim) * value_scale
                scores_fp4 = sum(q[row, heads].float() @ k.T for q in query_values) * score_scale
            else:
                scores_fp4, v = torch.zeros(ratio, 0), torch.zeros(0, dim)
            scores_tail = values_tail = scores_sink = values_sink = None
            if has_tail:
                qb = query_padded[row, heads].float()
                scores_tail = qb @ tail_key[slot, :PAGE, kvh].float().T
                values_tail = tail_value[slot, :PAGE, kvh]
                if has_sink:
                    scores_sink = qb @ tail_key[slot, PAGE:, kvh].float().T
                    values_sink = tail_value[slot, PAGE:, kvh]
            for part in range(parts):
                if num_splits == 1:
                    page_range, with_bf16 = None, True
                elif bf16_split:
                    page_range = split_page_range(pages, num_splits, part) if part < num_splits else (0, 0)
                    with_bf16 = part == num_splits
                    if with_bf16 and not has_tail:
                        continue
                else:
                    cost = bf16_page_cost if has_tail else 0
                    page_range, with_bf16 = split_page_range(pages, num_splits, part, cost), part == 0
                blocks = kernel_order_blocks(
                    scores_fp4=scores_fp4, values_fp4=v, fp4_tokens=fp4_tokens, scores_tail=scores_tail,
                    values_tail=values_tail, tail_tokens=tail_tokens, scores_sink=scores_sink,
                    values_sink=values_sink, sink_tokens=sink_tokens, page_range=page_range,
                    with_bf16=with_bf16)
                if bf16_split and num_splits > 1 and part == num_splits:
                    blocks = [b for b in blocks if b[2] == "bf16"]
                o, lse = online_attention(blocks, softmax_scale=softmax_scale, p_mode=p_mode, tau=tau,
                                          rescale_threshold=rescale_threshold, p_quantizer=p_quantizer)
                partial_out[part, row, heads] = o
                partial_lse[part, row, heads] = lse
    if parts == 1:
        return partial_out[0].to(torch.bfloat16), partial_out, partial_lse
    return combine_partials(partial_out, partial_lse), partial_out, partial_lse


def plain_attention(query: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, softmax_scale: float):
    """Exact FP32 softmax attention of ``[G,128]`` queries over ``[T,128]`` keys/values: the plain
    dequantise-then-attend result that the FP4-operand kernel is reported against."""
    scores = (query.float() @ keys.float().T) * softmax_scale
    return torch.softmax(scores, dim=-1) @ values.float()


def combine_partials(partial_out: torch.Tensor, partial_lse: torch.Tensor) -> torch.Tensor:
    """``[parts, ..., 128]`` FP32 + ``[parts, ...]`` LSE -> BF16, summing in part order under
    positive weights only (src/nvfp4_decode_kernel/split_k_combine.py:47-83)."""
    lse_max = partial_lse.amax(dim=0)
    lse_max = torch.where(torch.isinf(lse_max) & (lse_max < 0), torch.zeros_like(lse_max), lse_max)
    log2e = math.log2(math.e)
    weight = torch.exp2(partial_lse * log2e - lse_max * log2e)
    total = weight.sum(dim=0)
    inverse = torch.where((total == 0) | torch.isnan(total), torch.zeros_like(total), 1.0 / total)
    out = torch.zeros_like(partial_out[0])
    for s in range(partial_out.shape[0]):
        scale = weight[s] * inverse
        term = torch.where((scale > 0)[..., None], scale[..., None] * partial_out[s], torch.zeros_like(out))
        out = out + term
    return out.to(torch.bfloat16)
