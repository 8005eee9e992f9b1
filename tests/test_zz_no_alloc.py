"""The allocation-free split decode against the ordinary split decode, through the C ABI.

Some callers cannot allocate device memory at decode time (an engine whose allocator is frozen
after the KV cache took the HBM budget, a plugin entered while the framework holds its memory
pool). ``bdfp4_decode_split_static`` keeps the split path's partial buffers in a fixed array of
the library instead. This file is collected last on purpose: if it fails under ``-x``, every other
test has already run. It passes alone in a fresh process and after the other tests, because the
shared array needs no particular starting contents.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

# Both entry points run the same two kernels on the same inputs; only the address of the partial
# buffers differs. The outputs must therefore be identical, bit for bit: any tolerance here would
# let a stale partial of the shared array leak in at a small weight unnoticed.


def _args(w, quantized, padded, out, num_splits, bf16_split):
    import bdfp4
    from nvfp4_decode_kernel import _decode

    a = bdfp4.DecodeArgs()
    _decode._fill_args(
        a, rows=w.rows, heads_q=w.heads_q, heads_kv=w.heads_kv, page_count=w.regions[0].shape[0],
        query_fp4=quantized[0], query_scales=quantized[1], query_fp4_second=quantized[2],
        query_scales_second=quantized[3], query_padded_bf16=padded, key_pages_fp4=w.regions[0],
        key_scales=w.regions[1], value_pages_fp4=w.regions[2], value_scales=w.regions[3],
        fp4_page_table=w.page_table, seqused_fp4=w.seqused_fp4, residual_key_pages_bf16=w.tail_key[0],
        residual_value_pages_bf16=w.tail_value[0], residual_page_ids=w.slot_ids,
        seqused_residual=w.seqused_residual, seqused_sink=w.seqused_sink, softmax_scale=128 ** -0.5)
    a.num_splits, a.bf16_split = num_splits, int(bf16_split)
    a.out, a.out_row_stride = out.data_ptr(), out.stride(0)
    return a


def _both_ways(seed, seq_lens, num_splits, bf16_split, heads_q=8, heads_kv=2, with_tail=True):
    import bdfp4
    from bdfp4.workload import build_workload
    from nvfp4_decode_kernel._quantize import quantize_query

    w = build_workload(rows=len(seq_lens), heads_q=heads_q, heads_kv=heads_kv, seq_lens=seq_lens, sink_tokens=16,
                       seed=seed)
    padded = torch.zeros(w.rows, 128, w.heads_q, 128, dtype=torch.bfloat16, device="cuda")
    quantized = quantize_query(w.query, query_padded_out=padded, heads_kv=w.heads_kv, query_terms=2)
    stream = bdfp4.current_stream(w.device)
    # the caller-scratch path sizes its buffers for the extra BF16 part it asks for, used or not
    parts = num_splits + int(bf16_split)

    def strip_tail(a):
        if not with_tail:
            a.tail_key = a.tail_value = a.tail_slot_ids = a.seqused_residual = a.seqused_sink = None
        return a

    want = torch.empty(w.rows, w.heads_q, 128, dtype=torch.bfloat16, device="cuda")
    partial = torch.empty(parts * w.rows * w.heads_q * 128, device="cuda")
    lse = torch.empty(parts * w.rows * w.heads_q, device="cuda")
    a = strip_tail(_args(w, quantized, padded, want, num_splits, bf16_split))
    a.partial_out, a.partial_lse = partial.data_ptr(), lse.data_ptr()
    bdfp4.decode(a, stream)
    bdfp4.combine(partial, lse, parts, w.rows, w.heads_q, want, want.stride(0), stream)

    got = torch.full_like(want, float("nan"))
    b = strip_tail(_args(w, quantized, padded, got, num_splits, bf16_split))
    # a caller's counter array must not switch on a second, fused merge inside the static entry
    counters = torch.zeros(w.rows * w.heads_kv, dtype=torch.int32, device="cuda")
    b.merge_counters = counters.data_ptr()
    bdfp4.decode_split_static(b, stream)
    torch.cuda.synchronize()
    assert int(counters.abs().sum()) == 0
    return got, want


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    # two calls in a row, the second with fewer parts and rows than the first, so that it runs
    # over whatever the first one left in the shared array
    for seed, lens, splits, own in ((1, [1500, 260, 700], 4, True), (2, [300, 900], 2, False)):
        got, want = _both_ways(seed, lens, splits, own)
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)


def test_static_scratch_bf16_part_requested_without_a_tail():
    """bf16_split = 1 but no BF16 buffers: the static entry drops the part nothing would write (its
    stale log-sum-exp in the shared array would otherwise take part in the merge) and still agrees
    with the caller-scratch path, whose extra part reports itself empty."""
    got, want = _both_ways(3, [900, 400, 260], 3, True, with_tail=False)
    assert torch.isfinite(got.float()).all()
    assert torch.equal(got, want)


def test_static_scratch_largest_request_that_fits():
    """(parts * rows * heads_q) * 129 floats against the 2 Mi-float array: 127 rows x 32 heads x 4 parts
    (16,256 records) is the largest such batch that fits and must run; one more row must be refused."""
    import bdfp4

    got, want = _both_ways(4, [300] * 127, 4, False, heads_q=32, heads_kv=8, with_tail=False)
    assert torch.equal(got, want)
    a = bdfp4.DecodeArgs()
    a.rows, a.heads_q, a.heads_kv, a.num_splits = 128, 32, 8, 4
    a.out, a.out_row_stride = 16, 32 * 128  # never dereferenced: the size check comes first
    assert bdfp4.library().bdfp4_decode_split_static(ctypes.byref(a), None) == bdfp4.E_TOO_LARGE


def test_static_scratch_refuses_oversized_requests():
    import bdfp4

    a = bdfp4.DecodeArgs()
    a.rows, a.heads_q, a.heads_kv, a.num_splits = 4096, 32, 8, 8
    a.out, a.out_row_stride = 16, 32 * 128  # never dereferenced: the size check comes first
    status = bdfp4.library().bdfp4_decode_split_static(ctypes.byref(a), None)
    assert status == bdfp4.E_TOO_LARGE
    assert b"fixed-capacity" in bdfp4.library().bdfp4_status_string(status)
    a.num_splits = 1
    assert bdfp4.library().bdfp4_decode_split_static(ctypes.byref(a), None) == bdfp4.E_ARG
