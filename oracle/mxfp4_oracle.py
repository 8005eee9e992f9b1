"""CPU oracle of the MXFP4 format (E2M1 codes, one E8M0 power-of-two scale per 32 values).
TEST INFRASTRUCTURE: only tests may import it; the product never does.

Restates mxfp4_quantize and mxfp4_probability_quantize of OpenBitSys/BitDecoding-FP4
(src/nvfp4_decode_kernel/reference.py:262-358) and is pinned bit-exactly against outputs of those
functions in tests/golden/mxfp4_vectors.npz (made by tests/golden/make_mxfp4_golden.py).

    ocp       exponent = floor(log2(amax)) - 2, clamped to the E8M0 range [-127, 127]
    round_up  ocp + 1 when amax > 6 * 2^ocp (the smallest exponent keeping amax within E2M1's 6)
    search    ocp + 1 when it reconstructs the group with strictly less squared error
    an all-zero group takes exponent -127 (E8M0 has no zero); the stored byte is exponent + 127
"""

from __future__ import annotations

import torch

from . import nvfp4_oracle as base

GROUP = 32
RULES = ("ocp", "round_up", "search")
EXPONENT_MIN, EXPONENT_MAX = -127, 127


def _group_squares(difference: torch.Tensor) -> torch.Tensor:
    """Squared error of a 32-value group as the reference accumulates it: each half of sixteen by FMA in
    element order, then one FP32 sum of the halves (reference.py:113-118; the kernel's group is owned
    by two lanes)."""
    return base._fma_squares(difference[..., :16]) + base._fma_squares(difference[..., 16:])


def _power_of_two(exponent: torch.Tensor) -> torch.Tensor:
    return torch.ldexp(torch.ones(exponent.shape, dtype=torch.float32), exponent)


def _on_scale(groups: torch.Tensor, exponent: torch.Tensor):
    """Codes of ``groups`` on the scale ``2**exponent`` and the values they read back as."""
    scale = _power_of_two(exponent)
    codes = base.e2m1_codes(groups / scale)
    return codes, base.e2m1_decode(codes) * scale


def ocp_exponent(amax: torch.Tensor) -> torch.Tensor:
    """floor(log2(amax)) - 2 without a logarithm: amax = m * 2^k with m in [0.5, 1) gives
    floor(log2(amax)) = k - 1 (reference.py:299-306)."""
    _, k = torch.frexp(amax.float())
    exponent = (k.to(torch.int32) - 3).clamp(EXPONENT_MIN, EXPONENT_MAX)
    return torch.where(amax > 0, exponent, torch.full_like(exponent, EXPONENT_MIN))


def quantize_last_axis(x: torch.Tensor, rule: str = "ocp"):
    """``[..., n]`` (n % 32 == 0) -> (codes u8 ``[..., n]``, E8M0 bytes ``[..., n/32]``, winner
    int64 ``[..., n/32]``: 0 for the OCP exponent, 1 for the one above it)."""
    if rule not in RULES:
        raise ValueError(f"rule must be one of {RULES}, got {rule!r}")
    groups = x.float().reshape(*x.shape[:-1], x.shape[-1] // GROUP, GROUP)
    amax = groups.abs().amax(dim=-1, keepdim=True)
    exponent = ocp_exponent(amax)
    codes, values = _on_scale(groups, exponent)
    winner = torch.zeros_like(exponent, dtype=torch.int64)
    if rule != "ocp":
        above = (exponent + 1).clamp(max=EXPONENT_MAX)
        above_codes, above_values = _on_scale(groups, above)
        if rule == "round_up":
            choose = amax > 6.0 * _power_of_two(exponent)
        else:
            choose = (_group_squares(above_values - groups) < _group_squares(values - groups))[..., None]
        winner = choose.to(torch.int64)
        exponent = torch.where(choose, above, exponent)
        codes = torch.where(choose, above_codes, codes)
    return codes.reshape(x.shape), (exponent + 127).to(torch.uint8).squeeze(-1), winner.squeeze(-1)


def dequantize_last_axis(codes: torch.Tensor, scale_bytes: torch.Tensor) -> torch.Tensor:
    groups = base.e2m1_decode(codes).reshape(*codes.shape[:-1], codes.shape[-1] // GROUP, GROUP)
    scale = _power_of_two(scale_bytes.to(torch.int32) - 127)
    return (groups * scale[..., None]).reshape(codes.shape)


def probability_quantize(p: torch.Tensor):
    """The probability operand in MXFP4 (reference.py:331-358): start from ``round_up`` and take the
    exponent below it when that lowers ``mass^2 / 32 + sum of squared errors``, the error sums formed
    by a five-step pairwise (butterfly) reduction and the final combination in FP64 rounded to FP32.
    Returns (values the PV product sees, E8M0 bytes)."""
    codes, scale_bytes, _ = quantize_last_axis(p, "round_up")
    groups = p.float().reshape(*p.shape[:-1], p.shape[-1] // GROUP, GROUP)
    baseline = dequantize_last_axis(codes, scale_bytes).reshape(groups.shape)
    exponent = scale_bytes.to(torch.int32)[..., None] - 127
    below = (exponent - 1).clamp(min=EXPONENT_MIN)
    _, rival = _on_scale(groups, below)

    def cost(values):
        difference = values - groups
        squares, mass = difference.square(), difference
        for _ in range(5):
            squares = squares[..., 0::2] + squares[..., 1::2]
            mass = mass[..., 0::2] + mass[..., 1::2]
        return ((mass / 32).double() * mass.double() + squares.double()).float()

    choose = cost(rival) < cost(baseline)
    values = torch.where(choose, rival, baseline).reshape(p.shape)
    chosen = torch.where(choose, below, exponent).squeeze(-1)
    return values, (chosen + 127).to(torch.uint8)


# --------------------------------------------------------------------------------------
# page and query layouts (src/nvfp4_decode_kernel/quantize_kv_kernel.py:76-120,1040-1098 with
# sf_vec_size 32: one 512-byte atom of E8M0 bytes per (page, head), row r and group g < 4 at
# (r % 32) * 16 + (r // 32) * 4 + g; codes packed as for NVFP4)
# --------------------------------------------------------------------------------------

def atom_offsets() -> torch.Tensor:
    """``[128 rows, 4 groups]`` byte offsets inside one 512-byte scale atom."""
    r = torch.arange(128)[:, None]
    g = torch.arange(4)[None, :]
    return (r % 32) * 16 + (r // 32) * 4 + g


def _pack_atom(scale_bytes: torch.Tensor) -> torch.Tensor:
    """``[..., rows <= 128, 4]`` bytes -> ``[..., 512]`` (unused rows zero)."""
    rows = scale_bytes.shape[-2]
    atom = torch.zeros(*scale_bytes.shape[:-2], 512, dtype=torch.uint8)
    atom[..., atom_offsets()[:rows].reshape(-1)] = scale_bytes.reshape(*scale_bytes.shape[:-2], rows * 4)
    return atom


def _unpack_atom(atom: torch.Tensor, rows: int = 128) -> torch.Tensor:
    return atom[..., atom_offsets()[:rows].reshape(-1)].reshape(*atom.shape[:-1], rows, 4)


def quantize_key_pages(key_pages: torch.Tensor, rule: str = "ocp", *, rotate: bool = False, shift=None,
                       tensor_scale: float = 1.0):
    """``[pages, 128, H, 128]`` BF16 -> (codes u8 ``[pages,128,H,64]``, E8M0 atoms u8 ``[pages,H,512]``);
    groups of 32 along channels, after the NVFP4 path's cache-basis transform."""
    basis = base.divide_by_tensor_scale(base.key_cache_basis(key_pages, rotate=rotate, shift=shift), tensor_scale)
    codes, scale_bytes, _ = quantize_last_axis(basis.float(), rule)  # bytes [pages,tok,H,4]
    return base.pack_nibbles(codes), _pack_atom(scale_bytes.permute(0, 2, 1, 3))


def quantize_value_pages(value_pages: torch.Tensor, rule: str = "ocp", *, tensor_scale: float = 1.0):
    """``[pages, 128, H, 128]`` BF16 -> (codes u8 ``[pages,H,128,64]``, E8M0 atoms u8 ``[pages,H,512]``);
    groups of 32 along the page's tokens."""
    by_channel = base.divide_by_tensor_scale(value_pages.permute(0, 2, 3, 1), tensor_scale).float()
    codes, scale_bytes, _ = quantize_last_axis(by_channel, rule)  # bytes [pages,H,ch,4]
    return base.pack_nibbles(codes), _pack_atom(scale_bytes)


def dequantize_key_pages(codes: torch.Tensor, atoms: torch.Tensor) -> torch.Tensor:
    """-> FP32 ``[pages, 128, H, 128]``."""
    nib = base.unpack_nibbles(codes)  # [pages,tok,H,128]
    return dequantize_last_axis(nib, _unpack_atom(atoms).permute(0, 2, 1, 3))


def dequantize_value_pages(codes: torch.Tensor, atoms: torch.Tensor) -> torch.Tensor:
    nib = base.unpack_nibbles(codes)  # [pages,H,ch,tok]
    return dequantize_last_axis(nib, _unpack_atom(atoms)).permute(0, 3, 1, 2)


def quantize_query(query: torch.Tensor, heads_kv: int, *, rule: str = "ocp", terms: int = 1, rotate: bool = False,
                   tensor_scale: float = 1.0):
    """As ``nvfp4_oracle.quantize_query`` with E8M0 scales per 32: scale storage ``[rows,1,Hq,1,32,4,4]``,
    head ``h`` writing row ``h % G`` of the atom at head slot ``h // G``
    (src/nvfp4_decode_kernel/quantize_q_kernel.py:276-334 with ``is_mxfp4``)."""
    rows, heads_q, _ = query.shape
    ratio = heads_q // heads_kv
    values = base.hadamard_rotate(query) if rotate else query.float()
    out = {"padded": values.to(torch.bfloat16), "codes": [], "scales": [], "values": []}
    current = base.divide_by_tensor_scale(values, tensor_scale)
    offsets = atom_offsets()
    for _ in range(terms):
        codes, scale_bytes, _ = quantize_last_axis(current, rule)  # [rows,Hq,128], [rows,Hq,4]
        storage = torch.zeros(rows, heads_q, 512, dtype=torch.uint8)
        for h in range(heads_q):
            storage[:, h // ratio, offsets[h % ratio]] = scale_bytes[:, h]
        recon = dequantize_last_axis(codes, scale_bytes)
        out["codes"].append(base.pack_nibbles(codes).reshape(rows, 1, heads_q, 64))
        out["scales"].append(storage.reshape(rows, 1, heads_q, 1, 32, 4, 4))
        out["values"].append(recon)
        current = current - recon
    return out


def decode_reference(**kwargs):
    """``nvfp4_oracle.decode_reference`` over an MXFP4 cache: E8M0 pages, the MXFP4 probability operand
    (:func:`probability_quantize` per 32 tokens) and no ``c8`` shift (the reference builds the MXFP4
    kernel with rescale 0: src/nvfp4_decode_kernel/_decode.py:172-180). Parity of this composition is
    unpinned: the reference has no CPU model of whole MXFP4 attention, only of its pieces."""
    kwargs.setdefault("p_mode", "amax6")
    return base.decode_reference(dequantize_pages=(dequantize_key_pages, dequantize_value_pages),
                                 p_quantizer=lambda p: probability_quantize(p)[0], **kwargs)
