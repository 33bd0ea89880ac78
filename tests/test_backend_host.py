"""Host-side logic of B200Backend on CPU with a stub engine: block-table bookkeeping, page
allocation, and - where the reference checkout is present - the reference's own
ContinuousBatchScheduler driving the backend unchanged (the drop-in boundary)."""
import asyncio
import os
import sys

import pytest
import torch

from conftest import ROOT, pkg

# the reference checkout: a directory `reference` next to this repository unless REFERENCE_ROOT says otherwise
REF = os.environ.get("REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
HAVE_REF = os.path.isdir(os.path.join(REF, "src", "inference_server"))


class StubEngine:
    """Stands in for DecodeEngine: same static buffers, next token = current + 1 (as the reference's
    FakeBackend in tests/test_server.py), no arithmetic."""

    def __init__(self, num_blocks=64, max_batch=8, max_pages=16):
        self.cfg = pkg("engine").CONFIGS["tiny"]
        self.num_blocks, self.max_batch, self.max_pages = num_blocks, max_batch, max_pages
        self.device = torch.device("cpu")
        self.tokens = torch.zeros(max_batch, dtype=torch.int64)
        self.ctx_lens = torch.zeros(max_batch, dtype=torch.int32)
        self.block_table = torch.zeros(max_batch, max_pages, dtype=torch.int32)
        self.next_tokens = torch.zeros(max_batch, dtype=torch.int64)
        self.k_pools, self.v_pools, self._graphs = [], [], {}
        self.prefill_calls, self.steps = [], 0

    def step(self, B):
        self.next_tokens[:B] = self.tokens[:B] + 1
        self.ctx_lens[:B] += 1
        self.steps += 1
        return self.next_tokens[:B]

    def prefill(self, token_ids, block_ids, cached_tokens=0):
        assert len(block_ids) * 16 >= len(token_ids)
        self.prefill_calls.append((len(token_ids), cached_tokens))
        return token_ids[-1] + 1, None


def make_backend(**kw):
    return pkg("backend").B200Backend(StubEngine(**kw), max_new_tokens=8)


def test_prefill_reserves_pages_and_decode_keeps_row_order():
    be = make_backend()
    batch = None
    firsts = []
    for n in (5, 16, 33):
        kv, first, kv_len = be.prefill(list(range(100, 100 + n)), "s")
        assert kv_len == n and first == 100 + n and len(kv.block_ids) == (n + 8 + 15) // 16
        firsts.append(first)
        batch = be.splice_into_batched(batch, kv, kv_len)
    assert be.kv_length(batch) == 33
    nxt, batch = be.decode_step_batched(torch.tensor(firsts).view(-1, 1), batch, None, None)
    assert nxt.tolist() == [f + 1 for f in firsts] and nxt.device.type == "cpu"
    assert [r.ctx_len for r in batch.rows] == [6, 17, 34]
    eng = be.engine
    assert eng.ctx_lens[:3].tolist() == [6, 17, 34]  # engine advanced its own copy
    for i, row in enumerate(batch.rows):
        assert eng.block_table[i, : len(row.block_ids)].tolist() == row.block_ids


def test_remove_row_frees_private_pages_and_reorders_table():
    be = make_backend(num_blocks=12)
    batch = None
    for n in (20, 20, 20):  # 2 pages each (20 + 8 tokens)
        kv, _, _ = be.prefill(list(range(n)), "s")
        batch = be.splice_into_batched(batch, kv, n)
    assert len(be._alloc.free) == 12 - 6
    middle = list(batch.rows[1].block_ids)
    batch = be.remove_row_from_cache(batch, 1)
    assert len(batch.rows) == 2 and len(be._alloc.free) == 12 - 4
    assert set(middle) <= set(be._alloc.free)
    nxt, batch = be.decode_step_batched(torch.tensor([[7], [9]]), batch, None, None)
    assert nxt.tolist() == [8, 10]
    assert be.engine.block_table[1, :2].tolist() == batch.rows[1].block_ids


def test_decode_allocates_a_page_at_the_boundary_and_fails_cleanly_when_full():
    be = make_backend(num_blocks=2)
    be.max_new_tokens = 0
    kv, first, n = be.prefill(list(range(16)), "s")  # exactly one page, no reserve
    assert len(kv.block_ids) == 1
    batch = be.splice_into_batched(None, kv, n)
    nxt, batch = be.decode_step_batched(torch.tensor([[first]]), batch, None, None)
    assert len(batch.rows[0].block_ids) == 2  # token 17 needed a second page
    for _ in range(15):
        nxt, batch = be.decode_step_batched(nxt.view(1, 1), batch, None, None)
    with pytest.raises(MemoryError):
        be.decode_step_batched(nxt.view(1, 1), batch, None, None)


def test_chunked_prefill_primitives():
    be = make_backend()
    partial, matched = be.prefill_lookup(list(range(25)), "s")
    assert partial is None and matched == 0 and be.last_cache_hit_tokens == 0
    kv, last, n = be.prefill_chunk(list(range(0, 8)), None)
    kv, last, n = be.prefill_chunk(list(range(8, 25)), kv)
    assert n == 25 and last == 25 and be.engine.prefill_calls == [(8, 0), (25, 8)]
    be.prefill_store(list(range(25)), kv, 0, "s")  # no cache attached: a no-op


def test_generate_and_stream_stop_at_max_tokens_and_eos():
    be = make_backend()
    assert be.generate([1, 2, 3], 4) == [4, 5, 6, 7]
    be._eos_ids = {6}
    assert list(be.stream([1, 2, 3], 10)) == [4, 5]
    assert be.generate_batch([[1, 2], [10]], [2, 3]) == [[3, 4], [11, 12, 13]]
    assert len(be._alloc.free) == be.engine.num_blocks  # everything given back


@pytest.mark.skipif(not HAVE_REF, reason="reference checkout not present on this machine")
@pytest.mark.parametrize("chunk", [0, 8])
def test_reference_scheduler_drives_the_backend_unchanged(chunk):
    """ContinuousBatchScheduler (src/inference_server/scheduler.py) against B200Backend, as the reference's
    tests/test_chunked_prefill.py does with its fake backend: concurrent requests, admit/evict, token order."""
    sys.path.insert(0, os.path.join(REF, "src"))
    from inference_server.scheduler import ContinuousBatchScheduler, ScheduledRequest

    async def run():
        be = make_backend(num_blocks=256, max_batch=8, max_pages=32)
        sched = ContinuousBatchScheduler(be, max_batch_size=4, prefill_chunk_size=chunk)
        sched.start()
        try:
            loop = asyncio.get_running_loop()
            reqs = [ScheduledRequest(token_ids=list(range(10 * i, 10 * i + 5 + 7 * i)), max_tokens=3 + i,
                                     session_id=f"s{i}", future=loop.create_future()) for i in range(6)]
            outs = await asyncio.gather(*[sched.submit(r) for r in reqs])
            return be, outs, sched.stats()
        finally:
            await sched.stop()

    be, outs, stats = asyncio.run(run())
    for i, out in enumerate(outs):
        last = 10 * i + 5 + 7 * i - 1
        assert out == [last + 1 + j for j in range(3 + i)]
    assert stats["total_completed"] == 6
    assert len(be._alloc.free) == be.engine.num_blocks  # every page returned after eviction


@pytest.mark.skipif(not HAVE_REF, reason="reference checkout not present on this machine")
def test_reference_cache_manager_pools_and_prefix_hits_are_used_in_place():
    """With the reference's CacheManager attached (src/inference_server/kv_cache/cache_manager.py) the engine
    adopts its pools, a later prompt with a cached prefix gets the cached FULL pages as shared, read-only
    entries of its block table, and only the uncached suffix is run."""
    sys.path.insert(0, os.path.join(REF, "src"))
    from inference_server.kv_cache.cache_manager import CacheManager

    be = make_backend(num_blocks=64, max_batch=8, max_pages=16)
    cfg = be.engine.cfg
    cache = CacheManager(64, 16, layer_shapes=[(cfg.kv_heads, cfg.head_dim)] * cfg.layers, device="cpu",
                         dtype=torch.bfloat16)
    be.set_cache_adapter(cache)
    assert be.engine.k_pools is cache.block_manager.k_pools and be._alloc is None
    for p in cache.block_manager.k_pools:  # make stored pages recognisable
        p.copy_(torch.arange(p.numel(), dtype=torch.float32).reshape(p.shape) % 251)

    prompt_a = list(range(1000, 1040))  # 40 tokens = 2 full pages + 8
    kv_a, _, n_a = be.prefill(prompt_a, "a")
    assert n_a == 40 and be.last_cache_hit_tokens == 0 and be.engine.prefill_calls[-1] == (40, 0)
    stored = cache._exact_index[tuple(prompt_a)]
    assert [b.num_tokens_stored for b in stored] == [16, 16, 8]
    used_before = cache.block_manager.used_blocks

    prompt_b = prompt_a[:36] + [7, 8, 9, 10, 11]  # shares 36 tokens -> 2 full pages usable
    kv_b, _, n_b = be.prefill(prompt_b, "b")
    assert be.last_cache_hit_tokens == 32 and be.engine.prefill_calls[-1] == (41, 32)
    assert kv_b.block_ids[:2] == [stored[0].block_id, stored[1].block_id]  # shared pages, in place
    assert kv_b.block_ids[2] not in [b.block_id for b in stored]           # the tail page is private
    assert stored[0].ref_count >= 1                                        # protected while in use

    batch = be.splice_into_batched(None, kv_a, n_a)
    batch = be.splice_into_batched(batch, kv_b, n_b)
    nxt, batch = be.decode_step_batched(torch.tensor([[1], [2]]), batch, None, None)
    assert nxt.tolist() == [2, 3]
    be.remove_row_from_cache(batch, 1)
    be.remove_row_from_cache(batch, 0)
    cache.release(prompt_a, "a")
    cache.release(prompt_b, "b")
    # private pages went back to the reference allocator; cached prompt pages stay cached
    assert cache.block_manager.used_blocks <= used_before + 3
