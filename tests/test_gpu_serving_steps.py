"""Several serving steps through the plugin's device pieces, without a model: slot table, page
work table, tail reset, cache writer, decode with the fused tail write, and the promotion that
seals a filled tail page. A CPU model keeps every request's K/V history; after each step the
decode output is compared with the oracle and, at the end, the cache bytes with the oracle's
quantizer (bit-exact), including pages that were sealed from the BF16 tail."""

import pytest
import torch

from oracle import nvfp4_oracle as oracle

pytestmark = pytest.mark.gpu

HEADS_Q, HEADS_KV, LAYERS, SLOTS, BLOCKS, COLUMNS = 8, 2, 2, 4, 24, 5


class Request:
    def __init__(self, blocks, prompt, gen):
        self.blocks = blocks
        self.keys = [torch.randn(LAYERS, prompt, HEADS_KV, 128, generator=gen).to(torch.bfloat16)]
        self.values = [torch.randn(LAYERS, prompt, HEADS_KV, 128, generator=gen).to(torch.bfloat16)]
        self.new_tokens = prompt

    @property
    def length(self):
        return sum(k.shape[1] for k in self.keys)

    def append(self, gen):
        self.keys.append(torch.randn(LAYERS, 1, HEADS_KV, 128, generator=gen).to(torch.bfloat16))
        self.values.append(torch.randn(LAYERS, 1, HEADS_KV, 128, generator=gen).to(torch.bfloat16))
        self.new_tokens = 1

    def history(self, layer):
        return torch.cat([k[layer] for k in self.keys]), torch.cat([v[layer] for v in self.values])


def _oracle_row(request, layer, query, shift):
    """Oracle attention of one decode row over the request's whole history (this step's token
    included), with the cache's own split into sink / FP4 pages / rolling tail."""
    k, v = request.history(layer)
    n = k.shape[0]
    sink, fp4, tail = oracle.split_sequence_length(n)
    pages = fp4 // 128
    basis = oracle.key_cache_basis(k, rotate=True, shift=shift)
    kc, ks = oracle.quantize_key_pages(k[:fp4].reshape(pages, 128, HEADS_KV, 128), "four_six", rotate=True,
                                       shift=shift) if pages else (torch.zeros(1, 128, HEADS_KV, 64, dtype=torch.uint8),
                                                                   torch.zeros(1, HEADS_KV, 1024, dtype=torch.uint8))
    vc, vs = oracle.quantize_value_pages(v[:fp4].reshape(pages, 128, HEADS_KV, 128)) if pages else (
        torch.zeros(1, HEADS_KV, 128, 64, dtype=torch.uint8), torch.zeros(1, HEADS_KV, 1024, dtype=torch.uint8))
    tail_k = torch.zeros(1, 144, HEADS_KV, 128, dtype=torch.bfloat16)
    tail_v = torch.zeros_like(tail_k)
    tail_k[0, :tail], tail_v[0, :tail] = basis[fp4:], v[fp4:]
    tail_k[0, 128:128 + sink], tail_v[0, 128:128 + sink] = basis[:sink], v[:sink]
    q = oracle.quantize_query(query[None], HEADS_KV, terms=2, rotate=True)
    out, _, _ = oracle.decode_reference(
        query_values=q["values"], query_padded=q["padded"], key_codes=kc, key_scales=ks, value_codes=vc,
        value_scales=vs, page_table=torch.arange(max(pages, 1), dtype=torch.int32)[None],
        seqused_fp4=torch.tensor([fp4], dtype=torch.int32), heads_kv=HEADS_KV, softmax_scale=128 ** -0.5,
        tail_key=tail_k, tail_value=tail_v, tail_slot_ids=torch.zeros(1, dtype=torch.int32),
        seqused_residual=torch.tensor([tail], dtype=torch.int32), seqused_sink=torch.tensor([sink], dtype=torch.int32))
    return out[0]


def test_prefill_decode_promotion_and_slot_reuse():
    import types

    from nvfp4_vllm import layout, promote
    from nvfp4_vllm.control import ControlPlane
    from nvfp4_vllm.runtime import LayerRuntime
    from nvfp4_vllm.write import PageWorkTable, reset_new_request_tails, write_kv

    gen = torch.Generator().manual_seed(3)
    device = torch.device("cuda")
    plane = ControlPlane(max_num_seqs=SLOTS, max_num_batched_tokens=1024, device=device)
    table = PageWorkTable(max_num_seqs=SLOTS, max_num_batched_tokens=1024, device=device)
    runtime = LayerRuntime(num_layers=LAYERS, num_slots=SLOTS, num_heads=HEADS_Q, num_kv_heads=HEADS_KV,
                           head_dim=128, device=device, query_terms=2, rotation="hadamard",
                           key_scale_mode="four_six", value_scale_mode="amax6")
    runtime.key_shift = (0.2 * torch.randn(LAYERS, HEADS_KV, 128, generator=gen)).float().to(device)
    caches = [torch.zeros(BLOCKS, layout.page_bytes(HEADS_KV, 128), dtype=torch.uint8, device=device)
              for _ in range(LAYERS)]
    free_blocks = list(range(1, BLOCKS))

    def new_request(prompt):
        blocks = [free_blocks.pop(0) for _ in range(COLUMNS)]
        return Request(blocks, prompt, gen)

    def run_step(requests):
        """One engine step over `requests` (decode rows first, as the engine orders them)."""
        rows = sorted(requests, key=lambda r: r.new_tokens != 1)
        decode_rows = sum(1 for r in rows if r.new_tokens == 1)
        block_table = torch.zeros(SLOTS, COLUMNS, dtype=torch.int32)
        seq_lens = torch.zeros(SLOTS, dtype=torch.int32)
        qsl = torch.zeros(SLOTS + 1, dtype=torch.int32)
        for i, r in enumerate(rows):
            block_table[i] = torch.tensor(r.blocks)
            seq_lens[i] = r.length
            qsl[i + 1] = qsl[i] + r.new_tokens
        qsl[len(rows) + 1:] = qsl[len(rows)]
        tokens = int(qsl[len(rows)])
        block_table, seq_lens, qsl = block_table.to(device), seq_lens.to(device), qsl.to(device)
        outputs = plane.prepare(block_table=block_table, seq_lens=seq_lens[:len(rows)],
                                query_start_loc=qsl[:len(rows) + 1], num_reqs=len(rows), num_actual_tokens=tokens)
        max_query = max(r.new_tokens for r in rows)
        source_tokens, destination_pages = table.build(
            query_start_loc=qsl, seqused_fp4=outputs.seqused_fp4, row_to_slot=outputs.row_to_slot,
            block_table=block_table, num_reqs=len(rows), max_query_len=max_query)
        queries = torch.randn(decode_rows, HEADS_Q, 128, generator=gen).to(torch.bfloat16)
        results = []
        for layer in range(LAYERS):
            runtime.expect_layer(layer)
            key = torch.cat([r.keys[-1][layer] for r in rows]).to(device)
            value = torch.cat([r.values[-1][layer] for r in rows]).to(device)
            if layer == 0:
                reset_new_request_tails(tail_key=runtime.tail_key, tail_value=runtime.tail_value,
                                        query_start_loc=qsl[:len(rows) + 1], seq_lens=seq_lens[:len(rows)],
                                        row_to_slot=outputs.row_to_slot)
            raw_key, rotate_key, shift = runtime.key_write(layer, key)
            writer, regions = runtime.writer_for(layer, caches[layer])
            write_kv(writer=writer, regions=regions, key=raw_key, value=value, source_tokens=source_tokens,
                     destination_pages=destination_pages, query_start_loc=qsl[:len(rows) + 1],
                     seq_lens=seq_lens[:len(rows)], seqused_fp4=outputs.seqused_fp4,
                     row_to_slot=outputs.row_to_slot, layer_index=layer, decode_rows=decode_rows,
                     first_row=decode_rows if runtime.decode_writes_tail else 0)
            if decode_rows:
                # the call the plugin's attention layer makes for its decode rows
                step = types.SimpleNamespace(
                    row_to_slot=outputs.row_to_slot, seq_lens=seq_lens, seqused_fp4=outputs.seqused_fp4,
                    seqused_residual=outputs.seqused_residual, seqused_sink=outputs.seqused_sink,
                    block_table=block_table, decode_page_columns=COLUMNS, decode_num_splits=1, decode_row_order=None)
                out = torch.empty(decode_rows, HEADS_Q, 128, dtype=torch.bfloat16, device=device)
                runtime.attend_decode_rows(layer, decode_rows, query=queries.to(device), key=key, value=value,
                                           kv_cache=caches[layer], step=step, out=out, softmax_scale=128 ** -0.5,
                                           query_scale_mode="amax6")
                results.append(out.float().cpu())
                for i in range(decode_rows):
                    want = _oracle_row(rows[i], layer, queries[i], runtime.key_shift[layer].cpu())
                    err = (results[-1][i] - want.float()).abs()
                    assert float(err.max()) <= 1e-2, (layer, i, rows[i].length)
                    assert float(err.mean() / want.float().abs().mean()) <= 1e-3, (layer, i, rows[i].length)
            if layer == LAYERS - 1:
                metadata = type("M", (), dict(promotion_source_tokens=outputs.promotion_source_tokens,
                                              promotion_pages=outputs.promotion_pages))
                promote.launch(metadata, runtime)
        plane.raise_for_errors()

    a, b = new_request(250), new_request(126)
    run_step([a, b])                      # two prefills: a has one full page + tail, b only a tail
    for _ in range(4):                    # b's tail fills at 128 (promotion), a crosses 256 (promotion)
        a.append(gen)
        b.append(gen)
        run_step([a, b])
    c = new_request(300)                  # a mixed step: decode rows first, then a fresh prefill
    a.append(gen)
    b.append(gen)
    run_step([a, b, c])
    for _ in range(3):
        for r in (a, b, c):
            r.append(gen)
        run_step([a, b, c])
    # b finishes; d reuses b's blocks (a recycled key): its slot's tail must be cleared, not inherited
    d = Request(b.blocks, 40, gen)
    a.append(gen)
    c.append(gen)
    run_step([a, c, d])
    for r in (a, c, d):
        r.append(gen)
    run_step([a, c, d])

    # every sealed or prefilled page equals the oracle's quantization of the request's history
    torch.cuda.synchronize()
    for layer in range(LAYERS):
        blocks = caches[layer].cpu()
        kc = blocks[:, :8192 * HEADS_KV].reshape(-1, 128, HEADS_KV, 64)
        ks = blocks[:, 8192 * HEADS_KV:9216 * HEADS_KV].reshape(-1, HEADS_KV, 1024)
        vc = blocks[:, 9216 * HEADS_KV:17408 * HEADS_KV].reshape(-1, HEADS_KV, 128, 64)
        vs = blocks[:, 17408 * HEADS_KV:].reshape(-1, HEADS_KV, 1024)
        shift = runtime.key_shift[layer].cpu()
        for request in (a, c):
            k, v = request.history(layer)
            pages = ((request.length - 1) // 128)
            want_kc, want_ks = oracle.quantize_key_pages(k[:pages * 128].reshape(pages, 128, HEADS_KV, 128),
                                                         "four_six", rotate=True, shift=shift)
            want_vc, want_vs = oracle.quantize_value_pages(v[:pages * 128].reshape(pages, 128, HEADS_KV, 128))
            ids = torch.tensor(request.blocks[:pages])
            assert torch.equal(kc[ids], want_kc) and torch.equal(ks[ids], want_ks), (layer, request.length)
            assert torch.equal(vc[ids], want_vc) and torch.equal(vs[ids], want_vs), (layer, request.length)
