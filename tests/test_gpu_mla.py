"""MLA latent-cache path on the GPU against the CPU oracle (oracle/mla_oracle.py).

The reference has no MLA code, so nothing of the reference pins these results; the gates are
those of the GQA path: cache bytes and query codes bit-exact against the oracle's composition of
the pinned NVFP4 quantizer and page layouts, attention within max |err| <= 1e-2 and mean relative
error <= 1e-3 of the oracle's kernel-faithful result (the absolute bound relative to the value
where the value exceeds 1: the latent's outlier channels make outputs of magnitude 2-20).
"""

import pytest
import torch

from oracle import mla_oracle as oracle

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_REL = 1e-2, 1e-3
SCALE = 576 ** -0.5


def _tokens(tokens, seed, loud_prefix=0):
    gen = torch.Generator().manual_seed(seed)
    latent = torch.randn(tokens, 512, generator=gen)
    channels = torch.randperm(512, generator=gen)[:8]
    latent[:, channels] *= torch.exp(1.5 * torch.randn(8, generator=gen))
    rope = torch.randn(tokens, 64, generator=gen)
    if loud_prefix:  # old tokens whose scores tower over the newer ones: the running maximum moves late
        latent[:loud_prefix] *= 6.0
    return latent.to(torch.bfloat16), rope.to(torch.bfloat16)


def _build(seq_lens, heads, seed, loud_prefix=0, key_mode="amax6", value_mode="amax6"):
    """A cache written by the CUDA writers for rows of the given lengths, pages in shuffled order."""
    from nvfp4_decode_kernel import mla

    gen = torch.Generator().manual_seed(seed)
    pages_per_row = [-(-n // 64) for n in seq_lens]
    total = sum(pages_per_row)
    order = torch.randperm(total + 1, generator=gen)[:total] if total else torch.zeros(0, dtype=torch.long)
    table = torch.zeros(len(seq_lens), max(max(pages_per_row), 1), dtype=torch.int32)
    latents, ropes, sources, destinations = [], [], [], []
    cursor = offset = 0
    for row, n in enumerate(seq_lens):
        padded = pages_per_row[row] * 64
        latent, rope = _tokens(padded, seed * 100 + row, loud_prefix)
        latent[n:] = 0
        rope[n:] = 0
        latents.append(latent)
        ropes.append(rope)
        for page in range(pages_per_row[row]):
            table[row, page] = order[cursor]
            sources.append(offset + page * 64)
            destinations.append(int(order[cursor]))
            cursor += 1
        offset += padded
    latent = torch.cat(latents) if latents else torch.zeros(0, 512, dtype=torch.bfloat16)
    rope = torch.cat(ropes) if ropes else torch.zeros(0, 64, dtype=torch.bfloat16)
    cache = mla.MLACache.allocate(total + 1, "cuda")
    mla.write_pages(cache, latent.cuda(), rope.cuda(), torch.tensor(sources, dtype=torch.int32).cuda(),
                    torch.tensor(destinations, dtype=torch.int32).cuda(), key_scale_mode=key_mode,
                    value_scale_mode=value_mode)
    q_latent = torch.randn(len(seq_lens), heads, 512, generator=gen).to(torch.bfloat16)
    q_rope = torch.randn(len(seq_lens), heads, 64, generator=gen).to(torch.bfloat16)
    return dict(cache=cache, table=table, latent=latent, rope=rope, sources=sources, destinations=destinations,
                q_latent=q_latent, q_rope=q_rope, seq_lens=torch.tensor(seq_lens, dtype=torch.int32),
                key_mode=key_mode, value_mode=value_mode)


def _oracle_cache(w):
    """The oracle's own cache regions, indexed by physical page."""
    pages = w["cache"].pages
    count = len(w["sources"])
    by_page = w["latent"].reshape(count, 64, 512)
    kc, ks, vc, vs = oracle.quantize_pages(by_page, w["key_mode"], w["value_mode"])
    dest = torch.tensor(w["destinations"], dtype=torch.long)

    def scatter(t):
        full = torch.zeros(pages, *t.shape[1:], dtype=t.dtype)
        full[dest] = t
        return full

    rope = scatter(w["rope"].reshape(count, 64, 64))
    return scatter(kc), scatter(ks), scatter(vc), scatter(vs), rope


@pytest.mark.parametrize("modes", [("amax6", "amax6"), ("four_six", "amax6"), ("four_six_sixhalf", "four_six")])
def test_cache_bytes_are_the_oracles(modes):
    w = _build([200, 64, 333], 64, 7, key_mode=modes[0], value_mode=modes[1])
    kc, ks, vc, vs, rope = _oracle_cache(w)
    cache, dest = w["cache"], torch.tensor(w["destinations"], dtype=torch.long)
    got = {name: getattr(cache, name).cpu() for name in ("key_codes", "key_scales", "value_codes", "value_scales", "rope")}
    # a K page is head-major in memory: [4][64 tok][64 B]
    assert torch.equal(got["key_codes"][dest], kc.permute(0, 2, 1, 3).reshape(-1, 16384)[dest])
    assert torch.equal(got["key_scales"][dest], ks.reshape(-1, 2048)[dest])
    assert torch.equal(got["value_codes"][dest], vc.reshape(-1, 16384)[dest])
    assert torch.equal(got["value_scales"][dest], vs.reshape(-1, 2048)[dest])
    assert torch.equal(got["rope"][dest], oracle.rope_page_bytes(rope)[dest])


@pytest.mark.parametrize("mode", ["amax6", "four_six"])
def test_query_codes_are_the_oracles(mode):
    from nvfp4_decode_kernel import mla

    gen = torch.Generator().manual_seed(3)
    q = (torch.randn(5, 64, 512, generator=gen) * 3).to(torch.bfloat16)
    codes, scales = mla.quantize_query(q.cuda(), mode)
    want_codes, want_scales, _ = oracle.quantize_query(q, mode)
    assert torch.equal(codes.cpu(), want_codes)
    assert torch.equal(scales.cpu(), want_scales)


def _check(w, heads, num_splits=1, p_mode="amax2_or_amax6_c8"):
    from nvfp4_decode_kernel import mla

    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = mla.mla_decode(w["q_latent"].cuda(), w["q_rope"].cuda(), w["cache"], w["table"].cuda(),
                         w["seq_lens"].cuda(), softmax_scale=SCALE, num_splits=num_splits, p_scale_mode=p_mode,
                         error_word=error)
    torch.cuda.synchronize()
    assert int(error.item()) == 0
    kc, ks, vc, vs, rope = _oracle_cache(w)
    _, _, q_values = oracle.quantize_query(w["q_latent"])
    want, _, _ = oracle.decode_reference(q_values=q_values, q_rope=w["q_rope"], key_codes=kc, key_scales=ks,
                                         value_codes=vc, value_scales=vs, rope=rope, page_table=w["table"],
                                         seq_lens=w["seq_lens"], softmax_scale=SCALE, p_mode=p_mode,
                                         num_splits=num_splits)
    err = (out.float().cpu() - want.float()).abs()
    mean_rel = float(err.mean() / want.float().abs().mean().clamp_min(1e-6))
    # the latent's outlier channels carry outputs well above 1, where one BF16 step already exceeds
    # 1e-2: the absolute bound applies up to magnitude 1 and scales with the value above it
    excess = float((err - MAX_ABS * want.float().abs().clamp_min(1.0)).max())
    assert excess <= 0 and mean_rel <= MEAN_REL, (float(err.max()), excess, mean_rel)
    return out


@pytest.mark.parametrize("heads", [64, 128])
def test_decode_matches_the_oracle(heads):
    # whole steps, an odd page count, a ragged last page, a single token
    w = _build([512, 200, 64, 333, 1], heads, 11)
    _check(w, heads)


@pytest.mark.parametrize("p_mode", ["amax6", "amax2_or_amax6"])
def test_decode_probability_modes(p_mode):
    w = _build([384, 130], 64, 13)
    _check(w, 64, p_mode=p_mode)


def test_decode_rescales_when_the_maximum_moves_late():
    # the oldest tokens score far above the newer ones: the output accumulated in tensor memory is
    # rescaled in place near the end of the walk
    w = _build([640, 900], 128, 17, loud_prefix=40)
    _check(w, 128)


def test_one_row_at_the_benchmarked_length():
    # 32,768 tokens, 128 heads: the length the MLA bench line is quoted at (one row of its 64), with a
    # second short row so that the pair's barriers also see rows of very different lengths in one launch
    w = _build([32768, 192], 128, 23)
    _check(w, 128)


@pytest.mark.parametrize("num_splits", [2, 5])
def test_decode_split_and_merge(num_splits):
    w = _build([1024, 200, 64], 64, 19)
    _check(w, 64, num_splits=num_splits)


def test_decode_is_close_to_exact_attention():
    """Against FP32 attention over the unquantized tensors: the quantization error itself, loose."""
    w = _build([768], 64, 23)
    out = _check(w, 64)
    want = oracle.plain_attention(w["q_latent"][0], w["q_rope"][0], w["latent"][:768], w["rope"][:768], SCALE)
    err = (out[0].float().cpu() - want).abs()
    assert float(err.mean() / want.abs().mean()) < 0.2


def test_empty_row_and_argument_checks():
    from nvfp4_decode_kernel import mla

    w = _build([0, 128], 64, 29)
    out = _check(w, 64)
    assert float(out[0].float().abs().max()) == 0.0
    with pytest.raises(NotImplementedError):
        mla.mla_decode(w["q_latent"][:, :32].contiguous().cuda(), w["q_rope"][:, :32].contiguous().cuda(), w["cache"],
                       w["table"].cuda(), w["seq_lens"].cuda(), softmax_scale=SCALE)


@pytest.mark.parametrize("num_splits", [1, 3])
def test_decode_with_scratch_is_capturable_and_identical(num_splits):
    """Preallocated scratch and output: the same bytes as the allocating call, also when the whole
    step (query quantize, decode, merge; programmatic dependent launches) is replayed from a CUDA graph."""
    from nvfp4_decode_kernel import mla

    w = _build([640, 200], 128, 31)
    args = (w["q_latent"].cuda(), w["q_rope"].cuda(), w["cache"], w["table"].cuda(), w["seq_lens"].cuda())
    plain = mla.mla_decode(*args, softmax_scale=SCALE, num_splits=num_splits)
    scratch = mla.MLAScratch(2, 128, num_splits, "cuda")
    out = torch.zeros(2, 128, 512, dtype=torch.bfloat16, device="cuda")
    same = mla.mla_decode(*args, softmax_scale=SCALE, num_splits=num_splits, scratch=scratch, out=out)
    assert same is out and torch.equal(out, plain)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        mla.mla_decode(*args, softmax_scale=SCALE, num_splits=num_splits, scratch=scratch, out=out)  # warm
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            mla.mla_decode(*args, softmax_scale=SCALE, num_splits=num_splits, scratch=scratch, out=out)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, plain)
    with pytest.raises(ValueError):
        mla.mla_decode(*args, softmax_scale=SCALE, num_splits=num_splits + 1, scratch=scratch)


def test_append_requantizes_the_open_page():
    """One token per row and step: after every append the cache holds exactly the oracle's
    quantization of the row's tokens so far (the open page zero past the last token), across page
    boundaries, and decode over it meets the gate."""
    from nvfp4_decode_kernel import mla

    starts, steps, heads = [0, 70, 127], 70, 128
    rows = len(starts)
    streams = [_tokens(((s + steps + 63) // 64) * 64, 900 + r) for r, s in enumerate(starts)]
    max_pages = max(t[0].shape[0] // 64 for t in streams)
    gen = torch.Generator().manual_seed(41)
    table = torch.randperm(rows * max_pages + 1, generator=gen)[:rows * max_pages].to(torch.int32).reshape(rows, max_pages)
    cache = mla.MLACache.allocate(rows * max_pages + 1, "cuda")
    appender = mla.MLAAppender(rows, "cuda")
    open_latent = torch.zeros(rows, 64, 512, dtype=torch.bfloat16)
    open_rope = torch.zeros(rows, 64, 64, dtype=torch.bfloat16)
    for r, start in enumerate(starts):  # what a prefill would have left: whole pages in the cache, the rest staged
        latent, rope = streams[r]
        whole = start // 64
        if whole:
            mla.write_pages(cache, latent[:whole * 64].cuda(), rope[:whole * 64].cuda(),
                            (torch.arange(whole, dtype=torch.int32) * 64).cuda(), table[r, :whole].contiguous().cuda())
        open_latent[r, :start - whole * 64] = latent[whole * 64:start]
        open_rope[r, :start - whole * 64] = rope[whole * 64:start]
    appender.load_open_pages(open_latent.cuda(), open_rope.cuda())
    seq_lens = torch.tensor(starts, dtype=torch.int32, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    table_gpu = table.cuda()
    for step in range(steps):
        new_latent = torch.stack([streams[r][0][starts[r] + step] for r in range(rows)]).cuda()
        new_rope = torch.stack([streams[r][1][starts[r] + step] for r in range(rows)]).cuda()
        appender.append(cache, new_latent, new_rope, seq_lens, table_gpu, error_word=error)
        seq_lens += 1
    torch.cuda.synchronize()
    assert int(error.item()) == 0
    regions = {name: getattr(cache, name).cpu() for name in ("key_codes", "key_scales", "value_codes", "value_scales", "rope")}
    for r, start in enumerate(starts):
        length = start + steps
        pages = -(-length // 64)
        latent, rope = (t[:pages * 64].clone() for t in streams[r])
        latent[length:] = 0
        rope[length:] = 0
        kc, ks, vc, vs = oracle.quantize_pages(latent.reshape(pages, 64, 512))
        ids = table[r, :pages].long()
        assert torch.equal(regions["key_codes"][ids], kc.permute(0, 2, 1, 3).reshape(pages, 16384)), r
        assert torch.equal(regions["key_scales"][ids], ks.reshape(pages, 2048)), r
        assert torch.equal(regions["value_codes"][ids], vc.reshape(pages, 16384)), r
        assert torch.equal(regions["value_scales"][ids], vs.reshape(pages, 2048)), r
        assert torch.equal(regions["rope"][ids], oracle.rope_page_bytes(rope.reshape(pages, 64, 64))), r
    # decode over the appended cache against the oracle reading the same bytes
    q_latent = torch.randn(rows, heads, 512, generator=gen).to(torch.bfloat16)
    q_rope = torch.randn(rows, heads, 64, generator=gen).to(torch.bfloat16)
    out = mla.mla_decode(q_latent.cuda(), q_rope.cuda(), cache, table_gpu, seq_lens, softmax_scale=SCALE)
    total = cache.pages
    _, _, q_values = oracle.quantize_query(q_latent)
    want, _, _ = oracle.decode_reference(
        q_values=q_values, q_rope=q_rope,
        key_codes=regions["key_codes"].reshape(total, 4, 64, 64).permute(0, 2, 1, 3),
        key_scales=regions["key_scales"].reshape(total, 4, 512), value_codes=regions["value_codes"].reshape(total, 4, 128, 32),
        value_scales=regions["value_scales"].reshape(total, 4, 512),
        rope=base_rope_from_bytes(regions["rope"]), page_table=table, seq_lens=seq_lens.cpu(),
        softmax_scale=SCALE)
    err = (out.float().cpu() - want.float()).abs()
    assert float((err - MAX_ABS * want.float().abs().clamp_min(1.0)).max()) <= 0
    assert float(err.mean() / want.float().abs().mean()) <= MEAN_REL


def base_rope_from_bytes(blocks: torch.Tensor) -> torch.Tensor:
    """u8 ``[pages, 8192]`` swizzled rope blocks -> BF16 ``[pages, 64, 64]`` (the placement is its own inverse)."""
    from oracle import nvfp4_oracle as base

    pages = blocks.shape[0]
    raw = base._place_chunks(blocks.reshape(pages, 64, 128), (torch.arange(64) & 7)[None, :])
    return raw.contiguous().view(torch.bfloat16).reshape(pages, 64, 64)
