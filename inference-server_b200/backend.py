"""B200Backend: the reference's backend interface on paged KV instead of dense caches.

Mirrors ``InferenceBackend`` (src/inference_server/backends/base.py:10-138) and the
behaviour of ``TorchBackend`` (src/inference_server/backends/torch_backend.py) method
for method, so ``ContinuousBatchScheduler`` (src/inference_server/scheduler.py) can
drive it unchanged:

  reference (dense)                                this backend (paged)
  -----------------------------------------------  ------------------------------------
  per-row kv = HF DynamicCache [1,H,L,D]           ``SeqKV``: page ids + context length
  batched_kv = left-padded DynamicCache [B,H,S,D]  ``PagedBatch``: list of ``SeqKV`` rows
  splice_into_batched: re-pad + torch.cat          append a row          (:337-362)
  remove_row_from_cache: torch.cat without row     delete a row, free its private pages (:327-335)
  decode_step_batched: model(...) on dense cache   block table + graph replay (:305-322)
  kv_length: keys.shape[2]                         max context length    (:364)

The ``attention_mask`` and ``position_ids`` the scheduler passes
(scheduler.py:386-397) are accepted and ignored: context lengths are backend
state.  ``next_tokens`` comes back as a CPU tensor so the scheduler's per-row
``.item()`` (scheduler.py:399-402) costs one device read per step.

If a reference ``CacheManager`` is attached (``set_cache_adapter``,
base.py:16-18) and owns bf16 pools of the right shape, the engine reads and
writes those very pools (kv_cache/block_manager.py:33-49), prefix hits from
``lookup`` (kv_cache/cache_manager.py:41-80) are used in place as shared
read-only pages, and prompts are registered with ``store`` (:82-127) exactly as
TorchBackend does.  The manager may return a partially filled block in the middle
of a hit (:60-70); the kernels need every page but the last to be full, so the
leading full blocks are shared and the tokens from the first partial block on are
copied, compacted, into private pages of the row (no recomputation).  Without an
adapter the backend keeps its own free list.

The module has no CPU path for the arithmetic: constructing the engine needs a
CUDA device.  ``PagedBatch``/``SeqKV`` bookkeeping is plain Python and is what
the CPU tests exercise with a stub engine.
"""
from __future__ import annotations

import threading
import weakref
from dataclasses import dataclass, field
from typing import Generator

import torch

PAGE = 16


@dataclass
class SeqKV:
    """KV handle of one sequence: which pages hold it and how many tokens are valid."""

    block_ids: list[int]
    ctx_len: int
    private_blocks: list = field(default_factory=list)  # allocator handles this row must give back
    reserve_tokens: int = 0


@dataclass
class PagedBatch:
    """The opaque ``batched_kv`` the scheduler carries: rows in ``_active`` order."""

    rows: list[SeqKV] = field(default_factory=list)
    dirty: bool = True  # block table on the device needs a refresh


class _FreeListAllocator:
    """Page allocator used when no reference CacheManager is attached."""

    def __init__(self, num_blocks: int):
        self.free = list(range(num_blocks - 1, -1, -1))

    def allocate(self, n: int) -> list[int]:
        if n > len(self.free):
            raise MemoryError(f"Requested {n} blocks but only {len(self.free)} available")
        return [self.free.pop() for _ in range(n)]

    def release(self, ids: list[int]) -> None:
        self.free.extend(ids)


class B200Backend:
    """Implements the reference backend contract; see the module docstring."""

    cache_adapter = None
    last_cache_hit_tokens: int = 0

    def __init__(self, engine=None, eos_ids: set[int] | None = None, max_new_tokens: int = 256):
        self.engine = engine
        self._eos_ids: set[int] = set(eos_ids or ())
        self._lock = threading.Lock()  # the scheduler takes backend._lock (scheduler.py:184)
        self._alloc = _FreeListAllocator(engine.num_blocks) if engine is not None else None
        self.max_new_tokens = max_new_tokens
        self._table_cpu = None
        self._lens_cpu = None
        self._synced_batch = None  # the PagedBatch whose table is on the device right now
        self.status_check_every = 32  # decode steps between reads of the kernels' device status words
        self._steps_since_check = 0

    # ------------------------------------------------------------ lifecycle
    def set_cache_adapter(self, adapter) -> None:
        """Attach a reference CacheManager (base.py:16-18) and adopt its pools when they fit."""
        self.cache_adapter = adapter
        bm = getattr(adapter, "block_manager", None)
        eng = self.engine
        if bm is None or eng is None or not getattr(bm, "k_pools", None):
            return
        want = (eng.cfg.kv_heads, PAGE, eng.cfg.head_dim)
        ok = (len(bm.k_pools) == eng.cfg.layers and all(
            tuple(p.shape[1:]) == want and p.dtype == torch.bfloat16 and p.device.type == torch.device(eng.device).type
            for p in bm.k_pools))
        if not ok:
            raise ValueError("CacheManager pools do not match the engine (need bf16 pools on the engine's device, "
                             f"[num_blocks, {want[0]}, {want[1]}, {want[2]}] per layer, block_size 16)")
        eng.k_pools, eng.v_pools = bm.k_pools, bm.v_pools
        eng.num_blocks = bm.total_blocks
        eng.scratch_block = None  # the manager's pools have no spare page: graphs per exact batch size
        eng._graphs.clear()
        self._alloc = None  # pages now come from the reference BlockManager

    def load_model(self, model_name: str, num_blocks: int = 4096, max_batch: int = 64,
                   max_pages_per_seq: int = 256) -> None:
        """Load a Qwen3-MoE checkpoint as TorchBackend.load_model does (torch_backend.py:33-53):
        ``AutoModelForCausalLM.from_pretrained(model_name, dtype=bfloat16)``, EOS ids from the model
        config; the weights are then converted to the engine's run-time formats (``engine_from_hf``: dense
        weights bf16, experts e4m3 with 128x128 block scales - taken as stored when the checkpoint is FP8).
        One of the built-in shape names (``engine.CONFIGS``) builds a random-init engine of that shape
        instead, for benchmarks without a checkpoint.  Needs a CUDA device either way."""
        from . import engine as eng_mod

        if model_name in eng_mod.CONFIGS:
            self.engine = eng_mod.DecodeEngine(eng_mod.CONFIGS[model_name], num_blocks=num_blocks, max_batch=max_batch,
                                               max_pages_per_seq=max_pages_per_seq)
        else:
            model, self.tokenizer = self._read_checkpoint(model_name)
            eos = model.config.eos_token_id
            self._eos_ids = set(eos) if isinstance(eos, (list, tuple)) else ({eos} if eos is not None else set())
            self.engine = self._engine_from_model(model, num_blocks, max_batch, max_pages_per_seq)
            del model
        self._alloc = _FreeListAllocator(self.engine.num_blocks)
        self._table_cpu = self._lens_cpu = self._synced_batch = None
        if self.cache_adapter is not None:
            self.set_cache_adapter(self.cache_adapter)

    @staticmethod
    def _read_checkpoint(model_name: str):
        """(model on the host in bf16, tokenizer or None).  The tokenizer is optional here: the scheduler
        path passes token ids, and a checkpoint directory without tokenizer files still serves them."""
        from transformers import AutoModelForCausalLM, AutoTokenizer

        try:
            tok = AutoTokenizer.from_pretrained(model_name)
            if tok.pad_token is None:
                tok.pad_token = tok.eos_token
        except Exception:
            tok = None
        model = AutoModelForCausalLM.from_pretrained(model_name, dtype=torch.bfloat16)
        model.eval()
        return model, tok

    @staticmethod
    def _engine_from_model(model, num_blocks: int, max_batch: int, max_pages_per_seq: int):
        from . import engine as eng_mod

        return eng_mod.engine_from_hf(model, num_blocks=num_blocks, max_batch=max_batch,
                                      max_pages_per_seq=max_pages_per_seq)

    def enable_expert_parallel_rounds(self, group=None, idle_sleep: float = 0.002) -> None:
        """Data-parallel serving over an expert-parallel engine: every rank has its own scheduler and its own
        requests, yet each MoE layer of a pass exchanges rows with all ranks, so the ranks must run their passes
        in common rounds.  After this call every prompt chunk and decode step of this backend first agrees a
        round with the other ranks (``ep.RoundGate``), and a background thread answers, with an idle pass, the
        rounds that other ranks start while this one has nothing to run.  Collective: call it on every rank.
        The thread and the serving calls exclude each other through ``_lock``, which the scheduler holds for
        its whole tick (scheduler.py:184); direct callers of prefill / decode_step_batched must hold it too."""
        from . import ep

        if getattr(self.engine, "ep_state", None) is None:
            raise ValueError("the engine is not expert-parallel")
        self._round_keeper = ep.RoundKeeper(ep.RoundGate(group), self.engine.idle_pass, self._lock, idle_sleep).start()
        self.engine.round_hook = self._round_keeper.work_round

    def close(self) -> None:
        """Leave the expert-parallel rounds (the other ranks are told at their next round)."""
        keeper = getattr(self, "_round_keeper", None)
        if keeper is not None:
            keeper.close()
            self.engine.round_hook = None
            self._round_keeper = None

    def kv_shape_per_layer(self) -> list[tuple[int, int]]:
        cfg = self.engine.cfg
        return [(cfg.kv_heads, cfg.head_dim)] * cfg.layers

    @property
    def kv_dtype(self) -> torch.dtype:
        return torch.bfloat16

    @property
    def device(self):
        return self.engine.device

    @property
    def device_str(self) -> str:
        """The scheduler builds its token/mask tensors on this device (scheduler.py:173):
        host memory, so that they cost no device work."""
        return "cpu"

    def is_eos(self, token_id: int) -> bool:
        return token_id in self._eos_ids

    def kv_length(self, kv) -> int:
        if isinstance(kv, PagedBatch):
            return max((r.ctx_len for r in kv.rows), default=0)
        return kv.ctx_len

    # ---------------------------------------------------------------- pages
    def _take_pages(self, n: int) -> tuple[list[int], list]:
        if n <= 0:
            return [], []
        if self._alloc is not None:
            ids = self._alloc.allocate(n)
            return ids, ids
        bm = self.cache_adapter.block_manager
        # The manager evicts only from inside its own store() (cache_manager.py:93-98) and offers no public
        # call for it, because the reference keeps live sequences outside the pool.  Here live sequences sit in
        # pool pages, so room for them is made the way store() makes it: one unreferenced block at a time.
        evict = getattr(self.cache_adapter, "_evict_one", None)
        while n > bm.free_blocks:
            if evict is None or not evict():
                raise MemoryError(f"Requested {n} blocks but only {bm.free_blocks} available")
        blocks = bm.allocate(n)
        return [b.block_id for b in blocks], blocks

    def _give_back(self, handles: list) -> None:
        if not handles:
            return
        if self._alloc is not None:
            self._alloc.release(handles)
        else:
            self.cache_adapter.block_manager.free(handles)

    # -------------------------------------------------------------- prefill
    def _lookup(self, token_ids: list[int], session_id: str):
        """Prefix lookup as TorchBackend does (torch_backend.py:113-119).

        Returns (usable, shared_ids, tail, held): `usable` cached tokens can be skipped (always at least one
        token is left to run, so a full hit recomputes only its last token); the leading full blocks that lie
        wholly below `usable` are shared in place (`shared_ids`, still acquired); `tail` lists, for every
        further usable token, the (block id, slot) that holds its K/V - these come from a partially filled
        block in the middle of the hit or from the hit's last block, and the caller copies them into private
        pages; `held` are the acquired blocks behind `tail`, to release once the copy is queued."""
        cache = self.cache_adapter
        if cache is None or not getattr(cache.block_manager, "k_pools", None):
            return 0, [], [], []
        matched, blocks = cache.lookup(token_ids, session_id=session_id)
        usable = min(matched, len(token_ids) - 1)
        shared, tail, held = [], [], []
        pos, sharing = 0, True
        for blk in blocks:
            n = blk.num_tokens_stored
            if sharing and n == PAGE and pos + PAGE <= usable:
                shared.append(blk)
            else:
                sharing = False
                take = max(0, min(n, usable - pos))
                if take:
                    tail += [(blk.block_id, s) for s in range(take)]
                    held.append(blk)
                else:
                    blk.release()  # nothing of this block is used by the row
            pos += n
        return usable, [b.block_id for b in shared], tail, held

    def _adopt_tail(self, kv: SeqKV, first_pos: int, tail: list, held: list) -> None:
        """Copy the cached tokens listed in `tail` into the row's own pages at positions first_pos.. and let
        go of the blocks they came from."""
        try:
            if tail:
                dst = [(kv.block_ids[(first_pos + i) // PAGE], (first_pos + i) % PAGE) for i in range(len(tail))]
                self.engine.copy_kv_tokens(tail, dst)
        finally:
            for blk in held:
                blk.release()

    def _release_shared(self, shared_ids: list[int]) -> None:
        cache = self.cache_adapter
        if cache is None:
            return
        for bid in shared_ids:
            cache.block_manager.blocks[bid].release()

    def prefill(self, token_ids: list[int], session_id: str = "default"):
        """(per_row_kv, first_token_id, kv_length), as base.py:57-61.  Whatever raises on the way (a prompt
        wider than the block table, no pages left, a device finding) leaves no page and no block reference
        behind: the scheduler rejects the one request (scheduler.py:299-304) and carries on."""
        n = len(token_ids)
        total_pages = (n + self.max_new_tokens + PAGE - 1) // PAGE
        if n == 0:
            raise ValueError("prefill needs at least one token")
        if total_pages > self.engine.max_pages:
            raise ValueError(f"prompt of {n} tokens plus {self.max_new_tokens} reserved needs {total_pages} pages; "
                             f"the block table is {self.engine.max_pages} wide")
        matched, shared_ids, tail, held = self._lookup(token_ids, session_id)
        self.last_cache_hit_tokens = matched
        handles = []
        try:
            ids, handles = self._take_pages(total_pages - len(shared_ids))
            kv = SeqKV(block_ids=shared_ids + ids, ctx_len=n, private_blocks=handles)
            tail_blocks, held = held, []
            self._adopt_tail(kv, len(shared_ids) * PAGE, tail, tail_blocks)
            first, _ = self.engine.prefill(token_ids, kv.block_ids, cached_tokens=matched)
            self._check_status("prefill")
        except BaseException:
            for blk in held:
                blk.release()
            self._give_back(handles)
            self._release_shared(shared_ids)
            raise
        self._store(token_ids, kv, matched, session_id)
        return kv, first, n

    def _store(self, token_ids, kv: SeqKV, matched: int, session_id: str) -> None:
        """Register the prompt with the reference cache (torch_backend.py:143-145)."""
        cache = self.cache_adapter
        if cache is None or matched >= len(token_ids) or not getattr(cache.block_manager, "k_pools", None):
            return
        n = len(token_ids)
        n_pages = (n + PAGE - 1) // PAGE
        bt = torch.tensor(kv.block_ids[:n_pages], device=self.engine.device)
        per_layer = []
        for kp, vp in zip(self.engine.k_pools, self.engine.v_pools):
            k = kp[bt].permute(1, 0, 2, 3).reshape(kp.shape[1], n_pages * PAGE, kp.shape[3])[:, :n]
            v = vp[bt].permute(1, 0, 2, 3).reshape(vp.shape[1], n_pages * PAGE, vp.shape[3])[:, :n]
            per_layer.append((k, v))
        cache.store(token_ids, per_layer, skip_tokens=matched, session_id=session_id)

    def prefill_lookup(self, token_ids: list[int], session_id: str = "default"):
        matched, shared_ids, tail, held = self._lookup(token_ids, session_id)
        self.last_cache_hit_tokens = matched
        if matched == 0:
            return None, 0
        handles = []
        try:
            ids, handles = self._take_pages((matched + PAGE - 1) // PAGE - len(shared_ids))
            kv = SeqKV(block_ids=shared_ids + ids, ctx_len=matched, private_blocks=handles,
                       reserve_tokens=len(token_ids))
            tail_blocks, held = held, []
            self._adopt_tail(kv, len(shared_ids) * PAGE, tail, tail_blocks)
        except BaseException:
            for blk in held:
                blk.release()
            self._give_back(handles)
            self._release_shared(shared_ids)
            raise
        return kv, matched

    def prefill_chunk(self, chunk_token_ids: list[int], partial_kv):
        """Forward one chunk on top of partial_kv (base.py:71-78).  If the chunk cannot run, the pages taken
        for it go back; the partial KV of the earlier chunks stays as it was."""
        kv = partial_kv if partial_kv is not None else SeqKV(block_ids=[], ctx_len=0)
        new_len = kv.ctx_len + len(chunk_token_ids)
        total_pages = (new_len + self.max_new_tokens + PAGE - 1) // PAGE
        if total_pages > self.engine.max_pages:
            raise ValueError(f"{new_len} tokens plus {self.max_new_tokens} reserved need {total_pages} pages; "
                             f"the block table is {self.engine.max_pages} wide")
        ids, handles = self._take_pages(total_pages - len(kv.block_ids))
        try:
            # only the tokens past `cached_tokens` are embedded; the earlier ones are already pages
            tokens = [0] * kv.ctx_len + list(chunk_token_ids)
            last, _ = self.engine.prefill(tokens, kv.block_ids + ids, cached_tokens=kv.ctx_len)
            self._check_status("prefill_chunk")
        except BaseException:
            self._give_back(handles)
            raise
        kv.block_ids += ids
        kv.private_blocks += handles
        kv.ctx_len = new_len
        return kv, last, new_len

    def prefill_store(self, token_ids, full_kv, matched: int, session_id: str = "default") -> None:
        self._store(token_ids, full_kv, matched, session_id)

    # --------------------------------------------------------------- batching
    def _reclaim_rows(self, rows: list) -> None:
        for row in rows:
            self._give_back(row.private_blocks)
            row.private_blocks = []
        rows.clear()

    def splice_into_batched(self, batched_kv, new_kv, new_kv_len: int):
        if batched_kv is None:
            batch = PagedBatch()
            # The scheduler drops the whole batch object when its last row finishes
            # (scheduler.py:224-227) without calling remove_row_from_cache for it; give the pages of
            # whatever rows are still listed back when the batch object goes away.
            weakref.finalize(batch, self._reclaim_rows, batch.rows)
        else:
            batch = batched_kv
        batch.rows.append(new_kv)
        batch.dirty = True
        return batch

    def stack_caches_left_padded(self, per_row_caches: list, max_kv_len: int):
        batch = None
        for kv in per_row_caches:
            batch = self.splice_into_batched(batch, kv, kv.ctx_len)
        return batch

    def remove_row_from_cache(self, batched_kv, row_idx: int):
        row = batched_kv.rows.pop(row_idx)
        self._give_back(row.private_blocks)
        row.private_blocks = []
        batched_kv.dirty = True
        return batched_kv

    def _sync_table(self, batch: PagedBatch) -> int:
        eng = self.engine
        B = len(batch.rows)
        if B > eng.max_batch:
            raise ValueError(f"batch {B} exceeds the engine's max_batch {eng.max_batch}")
        # the device table belongs to the engine, not to a batch: a second live PagedBatch (generate_step with
        # separate caches, generate_batch beside the scheduler's batch) must re-upload even when it is clean
        if batch.dirty or self._table_cpu is None or self._synced_batch is None or self._synced_batch() is not batch:
            if self._table_cpu is None:
                pin = torch.cuda.is_available()
                self._table_cpu = torch.zeros(eng.max_batch, eng.max_pages, dtype=torch.int32, pin_memory=pin)
                self._lens_cpu = torch.zeros(eng.max_batch, dtype=torch.int32, pin_memory=pin)
            self._table_cpu.zero_()
            for i, row in enumerate(batch.rows):
                if len(row.block_ids) > eng.max_pages:
                    raise ValueError("sequence needs more pages than the block table is wide")
                self._table_cpu[i, : len(row.block_ids)] = torch.tensor(row.block_ids, dtype=torch.int32)
                self._lens_cpu[i] = row.ctx_len
            eng.block_table.copy_(self._table_cpu, non_blocking=True)
            eng.ctx_lens.copy_(self._lens_cpu, non_blocking=True)
            batch.dirty = False
            self._synced_batch = weakref.ref(batch)  # weak: a dropped batch must still give its pages back
        return B

    def _check_status(self, where: str) -> None:
        """Raise if a kernel recorded a finding (a block id outside the pool, a wait that ran out, an
        expert-parallel capacity overflow): such a step produced tokens from clamped or skipped data."""
        check = getattr(self.engine, "check_status", None)
        if check is not None:
            check(where)

    def decode_step_batched(self, current_tokens, batched_kv, attention_mask=None, position_ids=None):
        """One decode step for every row (base.py:89-99).  Returns (next_tokens [B] on the host, batched_kv)."""
        eng = self.engine
        batch: PagedBatch = batched_kv
        for row in batch.rows:
            if row.ctx_len + 1 > len(row.block_ids) * PAGE:
                ids, handles = self._take_pages(1)
                row.block_ids += ids
                row.private_blocks += handles
                batch.dirty = True
        B = self._sync_table(batch)
        tok = current_tokens.reshape(-1).to(torch.int64)
        eng.tokens[:B].copy_(tok, non_blocking=True)
        nxt = eng.step(B)
        out = nxt.to("cpu")  # synchronises: the scheduler reads every row right away
        for row in batch.rows:
            row.ctx_len += 1
        # The stream is idle after that read, so looking at the status words costs a few 4-byte copies; doing
        # it every few steps keeps a silent device finding from producing more than that many wrong tokens.
        self._steps_since_check += 1
        if self._steps_since_check >= self.status_check_every:
            self._steps_since_check = 0
            self._check_status("decode_step_batched")
        return out, batch

    def decode_step_with_prefill_chunk(self, current_tokens, batched_kv, chunk_token_ids: list[int], partial_kv,
                                       attention_mask=None, position_ids=None):
        """decode_step_batched and prefill_chunk as ONE pass over the model (base.py:89-99 and :71-78 together;
        the reference's scheduler runs them one after the other, scheduler.py:312-353 and :379-402, and its
        design notes name the merged pass as "Version B", docs/arch-scheduler.html:269-270).  The weights are
        streamed once for the decode rows and the chunk's tokens.
        Returns (next_tokens [B] on the host, batched_kv, kv, token after the chunk, new_len) - the two calls'
        results side by side.  If the pass cannot run, the pages taken for the chunk go back and neither the
        batch nor the partial KV has advanced."""
        eng = self.engine
        batch: PagedBatch = batched_kv
        kv = partial_kv if partial_kv is not None else SeqKV(block_ids=[], ctx_len=0)
        new_len = kv.ctx_len + len(chunk_token_ids)
        total_pages = (new_len + self.max_new_tokens + PAGE - 1) // PAGE
        if total_pages > eng.max_pages:
            raise ValueError(f"{new_len} tokens plus {self.max_new_tokens} reserved need {total_pages} pages; "
                             f"the block table is {eng.max_pages} wide")
        for row in batch.rows:
            if row.ctx_len + 1 > len(row.block_ids) * PAGE:
                ids, handles = self._take_pages(1)
                row.block_ids += ids
                row.private_blocks += handles
                batch.dirty = True
        ids, handles = self._take_pages(total_pages - len(kv.block_ids))
        try:
            B = self._sync_table(batch)
            tok = current_tokens.reshape(-1).to(torch.int64)
            eng.tokens[:B].copy_(tok, non_blocking=True)
            nxt, last, _ = eng.mixed_step(B, list(chunk_token_ids), kv.block_ids + ids, kv.ctx_len)
            out = nxt.to("cpu")
            self._check_status("decode_step_with_prefill_chunk")
        except BaseException:
            self._give_back(handles)
            batch.dirty = True  # the device lengths may have moved; re-upload them from the rows next time
            raise
        for row in batch.rows:
            row.ctx_len += 1
        kv.block_ids += ids
        kv.private_blocks += handles
        kv.ctx_len = new_len
        return out, batch, kv, last, new_len

    # ------------------------------------------- legacy whole-request entry points
    def generate(self, token_ids: list[int], max_tokens: int, template_prefix_len: int = 0,
                 session_id: str = "default") -> list[int]:
        return list(self.stream(token_ids, max_tokens, template_prefix_len, session_id))

    def stream(self, token_ids: list[int], max_tokens: int, template_prefix_len: int = 0,
               session_id: str = "default") -> Generator[int, None, None]:
        """Prefill then decode one sequence, yielding tokens (torch_backend.py:387-425 without the
        model-specific thinking-channel filter)."""
        with self._lock:
            kv, tok, _ = self.prefill(token_ids, session_id)
            batch = self.splice_into_batched(None, kv, kv.ctx_len)
            try:
                for _ in range(max_tokens):
                    if tok in self._eos_ids:
                        break
                    yield tok
                    nxt, batch = self.decode_step_batched(torch.tensor([[tok]]), batch)
                    tok = int(nxt[0])
            finally:
                self.remove_row_from_cache(batch, 0)
                if self.cache_adapter is not None:
                    self.cache_adapter.release(token_ids, session_id=session_id)

    def generate_batch(self, batch_token_ids: list[list[int]], max_tokens: list[int],
                       session_ids: list[str] | None = None) -> list[list[int]]:
        """Per-row prefill, batched decode (torch_backend.py:149-235)."""
        session_ids = session_ids or ["default"] * len(batch_token_ids)
        with self._lock:
            batch, cur = None, []
            for ids, sid in zip(batch_token_ids, session_ids):
                kv, first, n = self.prefill(ids, sid)
                batch = self.splice_into_batched(batch, kv, n)
                cur.append(first)
            out = [[] for _ in cur]
            done = [False] * len(cur)
            try:
                for _ in range(max(max_tokens)):
                    for i, t in enumerate(cur):
                        if done[i]:
                            continue
                        if t in self._eos_ids or len(out[i]) >= max_tokens[i]:
                            done[i] = True
                        else:
                            out[i].append(t)
                    if all(done):
                        break
                    nxt, batch = self.decode_step_batched(torch.tensor(cur).view(-1, 1), batch)
                    cur = [int(t) for t in nxt]
                return out
            finally:
                while batch is not None and batch.rows:
                    self.remove_row_from_cache(batch, 0)
                if self.cache_adapter is not None:
                    for ids, sid in zip(batch_token_ids, session_ids):
                        self.cache_adapter.release(ids, session_id=sid)

    def generate_step(self, token_ids: list[int], kv_cache=None):
        """Single step (base.py:41-45): prefill when there is no cache, else one decode step."""
        if kv_cache is None:
            kv, first, n = self.prefill(token_ids)
            return first, self.splice_into_batched(None, kv, n)
        nxt, batch = self.decode_step_batched(torch.tensor([[token_ids[-1]]]), kv_cache)
        return int(nxt[0]), batch
