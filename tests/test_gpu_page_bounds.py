"""Writers never follow a page id outside the cache: the item is skipped, the error word says so,
and the neighbouring pages keep their bytes. Nothing here faults: every id the kernels are given is
checked on the device before it is used as an address."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_kv_write_skips_destinations_past_the_cache():
    import bdfp4
    from bdfp4.workload import carve_cache
    from nvfp4_decode_kernel.quantize_kv_kernel import KVCacheWriter

    heads, pages = 2, 6
    blocks = torch.full((pages, 2 * 128 * heads * 72), 0xAB, dtype=torch.uint8, device="cuda")
    regions = carve_cache(blocks, heads)
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    writer = KVCacheWriter(regions=regions, key_scale_mode="four_six", error_word=error)
    gen = torch.Generator(device="cuda").manual_seed(0)
    key = torch.randn(4 * 128, heads, 128, generator=gen, device="cuda").to(torch.bfloat16)
    value = torch.randn(4 * 128, heads, 128, generator=gen, device="cuda").to(torch.bfloat16)
    source = torch.arange(4, dtype=torch.int32, device="cuda") * 128
    destination = torch.tensor([1, pages, -1, pages + 1000], dtype=torch.int32, device="cuda")
    writer(key, value, regions, source, destination)
    torch.cuda.synchronize()
    assert int(error.item()) & bdfp4.DEV_BAD_PAGE
    host = blocks.cpu()
    assert not bool((host[1] == 0xAB).all())             # the one valid item was written
    untouched = [0, 2, 3, 4, 5]
    assert bool((host[untouched] == 0xAB).all())         # nothing else was
    error.zero_()
    writer(key, value, regions, source[:1], destination[:1])
    torch.cuda.synchronize()
    assert int(error.item()) == 0


def test_mla_append_stops_at_the_last_table_column():
    """A row that has filled every column of its page table has no open page. One column further lies
    the next row's first entry, a valid page of another sequence: it must not be written."""
    import bdfp4
    from nvfp4_decode_kernel import mla

    rows, columns = 2, 2
    cache = mla.MLACache.allocate(8, "cuda")
    cache.blocks.fill_(0xCD)
    table = torch.tensor([[1, 2], [3, 4]], dtype=torch.int32, device="cuda")
    appender = mla.MLAAppender(rows, "cuda")
    seq_lens = torch.tensor([64 * columns, 5], dtype=torch.int32, device="cuda")  # row 0 is full
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(1)
    new_latent = torch.randn(rows, 512, generator=gen, device="cuda").to(torch.bfloat16)
    new_rope = torch.randn(rows, 64, generator=gen, device="cuda").to(torch.bfloat16)
    appender.append(cache, new_latent, new_rope, seq_lens, table, error_word=error)
    torch.cuda.synchronize()
    assert int(error.item()) & bdfp4.DEV_BAD_PAGE
    assert appender.destination_pages.tolist() == [-1, 3]
    host = cache.blocks.cpu()
    assert not bool((host[3] == 0xCD).all())             # row 1's open page was re-quantized
    assert bool((host[[0, 1, 2, 4, 5, 6, 7]] == 0xCD).all())  # row 0's token went to no page at all
