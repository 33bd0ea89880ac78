"""CUDA graphs of the decode step per batch bucket (B200): a batch of 3 runs the 4-row graph with one padding
row on the scratch page; the real rows get exactly what a graph of their own size gives, and nothing outside the
rows' own pages and the scratch page is written - in particular not by the warm-up runs of a graph build."""
import pytest
import torch

from conftest import pkg

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make(eng_mod, buckets):
    return eng_mod.DecodeEngine(eng_mod.CONFIGS["tiny"], num_blocks=32, max_batch=8, max_pages_per_seq=4, device=DEV,
                                seed=5, graph_buckets=buckets, keep_logits=True)


def test_bucketed_graph_equals_exact_graph_and_keeps_off_foreign_pages(ops):
    eng_mod = pkg("engine")
    a, b = make(eng_mod, True), make(eng_mod, False)
    assert a.scratch_block == 32 and a.k_pools[0].shape[0] == 33
    assert b.scratch_block is None and b.k_pools[0].shape[0] == 32
    assert [a.graph_batch(n) for n in (1, 2, 3, 4, 5, 8)] == [1, 2, 4, 4, 8, 8] and b.graph_batch(3) == 3
    B = 3
    g = torch.Generator().manual_seed(0)
    for e in (a, b):
        for li in range(e.cfg.layers):
            kv = torch.randn(32, *e.k_pools[li].shape[1:], generator=g).bfloat16().to(DEV)
            e.k_pools[li][:32].copy_(kv)
            e.v_pools[li][:32].copy_(kv.flip(0))
        g = torch.Generator().manual_seed(0)  # the same pool image in both engines
    # rows 0..2 own pages (1,2) (3,4) (5,6); lengths 15, 16, 30: row 0's next token fills its first page, row 1's
    # opens its second page, row 2 sits two tokens before the end of its last page
    for e in (a, b):
        e.block_table.zero_()
        for r in range(B):
            e.block_table[r, 0], e.block_table[r, 1] = 1 + 2 * r, 2 + 2 * r
        e.ctx_lens[:B] = torch.tensor([15, 16, 30], dtype=torch.int32)
        e.tokens[:B] = torch.tensor([11, 22, 33])
    before = [p.clone() for p in a.k_pools]
    outs = {}
    for name, e in (("bucket", a), ("exact", b)):
        toks = []
        for step in range(2):
            nxt = e.step(B).clone()
            e.tokens[:B].copy_(nxt)
            toks.append(nxt)
        torch.cuda.synchronize()
        e.check_status(name)
        outs[name] = (torch.stack(toks), e.last_logits[:B].clone())
    assert torch.equal(outs["bucket"][0], outs["exact"][0])
    assert torch.equal(outs["bucket"][1], outs["exact"][1])
    assert a.ctx_lens[:B].tolist() == [17, 18, 32] and sorted(a._graphs) == [4] and sorted(b._graphs) == [3]
    # few rows get their own (shorter) attention split and workspace; the full batch keeps the engine's
    assert set(a._attn_by_rows) == {4, 8} and a._attn_by_rows[8][1] is a.attn_ws
    # pages of the real rows are identical in both engines; no other page changed - block 0 (what an unallocated
    # table entry points to) included; only the scratch page of the bucketed engine was written
    for li in range(a.cfg.layers):
        assert torch.equal(a.k_pools[li][:32], b.k_pools[li][:32])
        changed = (a.k_pools[li][:32] != before[li][:32]).flatten(1).any(1).nonzero().flatten().tolist()
        assert set(changed) <= {1, 2, 3, 4, 6}, changed  # slots 15,16 / 16,17 / 30,31 of the rows' own pages
        assert bool((a.k_pools[li][32] != 0).any())
