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

    def copy_kv_tokens(self, src, dst):  # the engine's own (index arithmetic on the pools, any device)
        return pkg("engine").DecodeEngine.copy_kv_tokens(self, src, dst)


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


# ------------------------------------------------- failure paths and bookkeeping ----
class FailingEngine(StubEngine):
    """Refuses every prompt pass after the pages were taken, as a device finding or a full table would."""

    def prefill(self, token_ids, block_ids, cached_tokens=0):
        raise RuntimeError("engine refused the prompt")


def test_a_refused_prompt_leaves_no_pages_behind():
    be = pkg("backend").B200Backend(FailingEngine(num_blocks=32), max_new_tokens=8)
    with pytest.raises(RuntimeError, match="refused"):
        be.prefill(list(range(40)), "s")
    assert len(be._alloc.free) == 32
    with pytest.raises(RuntimeError, match="refused"):
        be.prefill_chunk(list(range(20)), None)
    assert len(be._alloc.free) == 32


def test_a_prompt_wider_than_the_block_table_is_refused_before_any_page_is_taken():
    be = make_backend(num_blocks=64, max_pages=4)  # 64 tokens per sequence at most
    with pytest.raises(ValueError, match="block table"):
        be.prefill(list(range(60)), "s")  # 60 + 8 reserved = 68 tokens = 5 pages
    assert len(be._alloc.free) == 64 and be.engine.prefill_calls == []
    kv, _, _ = be.prefill_chunk(list(range(40)), None)
    with pytest.raises(ValueError, match="block table"):
        be.prefill_chunk(list(range(40, 60)), kv)
    assert kv.ctx_len == 40 and len(kv.block_ids) == 3  # the earlier chunks are untouched


def test_two_live_batches_do_not_read_each_others_table():
    be = make_backend()
    kv1, f1, n1 = be.prefill(list(range(5)), "a")
    kv2, f2, n2 = be.prefill(list(range(50, 70)), "b")
    b1 = be.splice_into_batched(None, kv1, n1)
    b2 = be.splice_into_batched(None, kv2, n2)
    be.decode_step_batched(torch.tensor([[f1]]), b1, None, None)
    be.decode_step_batched(torch.tensor([[f2]]), b2, None, None)
    # b1 is clean (nothing admitted or evicted since its last step), yet the device table holds b2's row
    be.decode_step_batched(torch.tensor([[f1 + 1]]), b1, None, None)
    assert be.engine.block_table[0, : len(kv1.block_ids)].tolist() == kv1.block_ids
    assert int(be.engine.ctx_lens[0]) == 7


def test_device_findings_surface_on_the_serving_path():
    class Noting(StubEngine):
        checks, bad = 0, False

        def check_status(self, where):
            self.checks += 1
            if self.bad:
                raise RuntimeError(f"{where}: device: block table entry outside the pool")

    be = pkg("backend").B200Backend(Noting(), max_new_tokens=8)
    be.status_check_every = 4
    kv, first, n = be.prefill(list(range(5)), "s")
    assert be.engine.checks == 1  # right after the prompt pass
    batch = be.splice_into_batched(None, kv, n)
    tok = torch.tensor([[first]])
    for _ in range(3):
        tok, batch = be.decode_step_batched(tok.view(1, 1), batch, None, None)
    assert be.engine.checks == 1
    be.engine.bad = True
    with pytest.raises(RuntimeError, match="outside the pool"):
        be.decode_step_batched(tok.view(1, 1), batch, None, None)


@pytest.mark.skipif(not HAVE_REF, reason="reference checkout not present on this machine")
def test_a_partial_block_in_the_middle_of_a_hit_is_compacted_not_dropped():
    """The reference stores a prompt suffix in fresh blocks (cache_manager.py:82-127), so a prompt that was
    extended twice is cached as blocks of 16 + 6 + 11 tokens.  A hit on it shares the full leading block in
    place and copies the other 17 tokens, compacted, into the new row's own pages - none is recomputed."""
    sys.path.insert(0, os.path.join(REF, "src"))
    from inference_server.kv_cache.cache_manager import CacheManager

    be = make_backend(num_blocks=64, max_batch=8, max_pages=16)
    cfg = be.engine.cfg
    cache = CacheManager(64, 16, layer_shapes=[(cfg.kv_heads, cfg.head_dim)] * cfg.layers, device="cpu",
                         dtype=torch.bfloat16)
    be.set_cache_adapter(cache)
    p1 = list(range(500, 522))            # 22 tokens -> blocks of 16 + 6
    p2 = p1 + list(range(900, 911))       # + 11 -> a third block of 11
    p3 = p2 + [1, 2, 3, 4, 5]
    kv1, _, _ = be.prefill(p1, "a")
    kv2, _, _ = be.prefill(p2, "b")
    assert be.last_cache_hit_tokens == 22 and be.engine.prefill_calls[-1] == (33, 22)
    blocks = cache._exact_index[tuple(p2)]
    assert [b.num_tokens_stored for b in blocks] == [16, 6, 11]
    # make every cached token recognisable: value = 100 * block + slot, in every layer
    for kp, vp in zip(cache.block_manager.k_pools, cache.block_manager.v_pools):
        for b in blocks:
            for s in range(b.num_tokens_stored):
                kp[b.block_id, :, s, :] = 100 * b.block_id + s
                vp[b.block_id, :, s, :] = -(100 * b.block_id + s)
    refs_before = [b.ref_count for b in blocks]
    kv3, _, n3 = be.prefill(p3, "c")
    assert be.last_cache_hit_tokens == 33 and be.engine.prefill_calls[-1] == (38, 33)
    assert kv3.block_ids[0] == blocks[0].block_id                       # the full block is shared in place
    assert not set(kv3.block_ids[1:]) & {b.block_id for b in blocks}    # everything after it is private
    where = [(blocks[1].block_id, s) for s in range(6)] + [(blocks[2].block_id, s) for s in range(11)]
    kp, vp = cache.block_manager.k_pools[-1], cache.block_manager.v_pools[-1]
    for i, (b, s) in enumerate(where):
        pos = 16 + i
        got_k = kp[kv3.block_ids[pos // 16], :, pos % 16, :]
        got_v = vp[kv3.block_ids[pos // 16], :, pos % 16, :]
        assert bool((got_k == 100 * b + s).all()) and bool((got_v == -(100 * b + s)).all())
    # only the shared block stays acquired for the row; the copied-from blocks were let go again
    assert blocks[0].ref_count == refs_before[0] + 1
    assert [b.ref_count for b in blocks[1:]] == refs_before[1:]

    # an exact repeat of a cached prompt recomputes only its last token
    kv4, _, _ = be.prefill(p2, "d")
    assert be.last_cache_hit_tokens == 32 and be.engine.prefill_calls[-1] == (33, 32)


@pytest.mark.skipif(not HAVE_REF, reason="reference checkout not present on this machine")
def test_a_refused_prompt_lets_go_of_its_cache_hit():
    sys.path.insert(0, os.path.join(REF, "src"))
    from inference_server.kv_cache.cache_manager import CacheManager

    be = make_backend(num_blocks=64, max_batch=8, max_pages=16)
    cfg = be.engine.cfg
    cache = CacheManager(64, 16, layer_shapes=[(cfg.kv_heads, cfg.head_dim)] * cfg.layers, device="cpu",
                         dtype=torch.bfloat16)
    be.set_cache_adapter(cache)
    prompt = list(range(700, 740))
    be.prefill(prompt, "a")
    blocks = cache._exact_index[tuple(prompt)]
    refs, free = [b.ref_count for b in blocks], cache.block_manager.free_blocks

    def refuse(*a, **k):
        raise RuntimeError("engine refused the prompt")

    be.engine.prefill = refuse
    with pytest.raises(RuntimeError, match="refused"):
        be.prefill(prompt + [1, 2, 3], "b")
    assert [b.ref_count for b in blocks] == refs and cache.block_manager.free_blocks == free


def test_load_model_reads_a_checkpoint_as_the_reference_does(tmp_path, monkeypatch):
    """load_model(path) follows TorchBackend.load_model (torch_backend.py:33-53): from_pretrained in bf16, EOS ids
    from the model config (a list or a single id).  The conversion to run-time formats needs a GPU, so the engine
    constructor is replaced by one that records what it was handed."""
    from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM

    cfg = Qwen3MoeConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_experts=4,
                         num_experts_per_tok=2, moe_intermediate_size=32, decoder_sparse_step=1, mlp_only_layers=[],
                         eos_token_id=[5, 7], tie_word_embeddings=False)
    torch.manual_seed(0)
    Qwen3MoeForCausalLM(cfg).save_pretrained(tmp_path)
    seen = {}

    def fake_engine(model, num_blocks, max_batch, max_pages_per_seq):
        seen["dtype"] = next(model.parameters()).dtype
        seen["layers"] = len(model.model.layers)
        seen["experts"] = tuple(model.model.layers[0].mlp.experts.gate_up_proj.shape)
        return StubEngine(num_blocks=num_blocks, max_batch=max_batch, max_pages=max_pages_per_seq)

    be_cls = pkg("backend").B200Backend
    monkeypatch.setattr(be_cls, "_engine_from_model", staticmethod(fake_engine))
    be = be_cls(max_new_tokens=8)
    be.load_model(str(tmp_path), num_blocks=40, max_batch=4, max_pages_per_seq=8)
    assert seen == {"dtype": torch.bfloat16, "layers": 1, "experts": (4, 64, 64)}
    assert be._eos_ids == {5, 7} and be.is_eos(7) and not be.is_eos(6)
    assert be.engine.num_blocks == 40 and len(be._alloc.free) == 40
    kv, first, n = be.prefill([1, 2, 3], "s")  # the loaded backend serves requests
    assert n == 3 and first == 4
    with pytest.raises(Exception):
        be.load_model(str(tmp_path / "missing"))


class MixedStub(StubEngine):
    """StubEngine with the merged pass: decode rows as in step(), chunk's next token = last token + 1."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.mixed_calls, self.fail = [], False

    def mixed_step(self, B, chunk_token_ids, block_ids, first_pos, want_first=True):
        if self.fail:
            raise RuntimeError("engine refused the mixed pass")
        assert len(block_ids) * 16 >= first_pos + len(chunk_token_ids)
        self.mixed_calls.append((B, len(chunk_token_ids), first_pos))
        return self.step(B), chunk_token_ids[-1] + 1, None


def test_merged_decode_and_prompt_chunk_equals_the_two_calls():
    """decode_step_with_prefill_chunk leaves the batch, the partial KV and the allocator exactly where
    prefill_chunk followed by decode_step_batched leaves them (the reference's order, scheduler.py:312-402)."""
    prompts = [list(range(100, 120)), list(range(300, 333))]
    new = list(range(500, 540))

    def serve(merged):
        be = pkg("backend").B200Backend(MixedStub(), max_new_tokens=8)
        batch, toks = None, []
        for i, p in enumerate(prompts):
            kv, first, n = be.prefill(p, f"s{i}")
            batch = be.splice_into_batched(batch, kv, n)
            toks.append(first)
        tok = torch.tensor(toks).view(-1, 1)
        partial, outs = None, []
        for lo in range(0, len(new), 16):
            piece = new[lo:lo + 16]
            if merged:
                nxt, batch, partial, last, n = be.decode_step_with_prefill_chunk(tok, batch, piece, partial)
            else:
                partial, last, n = be.prefill_chunk(piece, partial)
                nxt, batch = be.decode_step_batched(tok, batch, None, None)
            outs.append((nxt.tolist(), last, n))
            tok = nxt.view(-1, 1)
        state = ([(r.block_ids, r.ctx_len) for r in batch.rows], partial.block_ids, partial.ctx_len,
                 sorted(be._alloc.free))
        return outs, state, be

    outs_a, state_a, _ = serve(False)
    outs_b, state_b, be = serve(True)
    assert outs_a == outs_b and state_a == state_b
    assert be.engine.mixed_calls == [(2, 16, 0), (2, 16, 16), (2, 8, 32)]


def test_a_refused_merged_pass_gives_the_chunks_pages_back():
    be = pkg("backend").B200Backend(MixedStub(num_blocks=32), max_new_tokens=8)
    kv, first, n = be.prefill(list(range(5)), "s")
    batch = be.splice_into_batched(None, kv, n)
    free = len(be._alloc.free)
    be.engine.fail = True
    with pytest.raises(RuntimeError, match="refused"):
        be.decode_step_with_prefill_chunk(torch.tensor([[first]]), batch, list(range(20)), None)
    assert len(be._alloc.free) == free and batch.rows[0].ctx_len == n
    be.engine.fail = False
    nxt, batch, partial, last, m = be.decode_step_with_prefill_chunk(torch.tensor([[first]]), batch, list(range(20)), None)
    assert int(nxt[0]) == first + 1 and last == 20 and m == 20 and batch.rows[0].ctx_len == n + 1
