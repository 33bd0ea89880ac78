"""Prompt pass through the paged kernels (B200): chunking and cached prefixes do not change the result.

`DecodeEngine.prefill` runs a prompt as rows of the decode kernels (one row per prompt token, shared block
table, per-row context length), so the KV pages are read in place.  Agreement with the reference model itself
is covered by tests/test_gpu_tiny_model.py (its prompts go through this function); here the properties that
make the path usable for chunked prefill and prefix-cache hits are checked."""
import pytest
import torch

from conftest import pkg, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
# Whole-model logits (2 layers + lm_head, bf16 activations): different chunkings change GEMM shapes, split
# boundaries and expert grouping, i.e. bf16 rounding points, not arithmetic.  The per-kernel bound is 1e-2.
TOL_MODEL = 3e-2


def make_engine():
    eng = pkg("engine")
    return eng.DecodeEngine(eng.CONFIGS["tiny"], num_blocks=64, max_batch=4, max_pages_per_seq=16, device=DEV, seed=3,
                            keep_logits=True)


def test_chunked_prefill_equals_one_pass_and_cached_prefix_is_read_in_place(ops):
    engine = make_engine()
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, 4096, (150,), generator=g).tolist()
    blocks = list(range(5, 15))  # 10 pages
    first_a, logits_a = engine.prefill(prompt, blocks, chunk=256)
    k_a = [p[blocks].clone() for p in engine.k_pools]
    for p in engine.k_pools + engine.v_pools:
        p.zero_()
    first_b, logits_b = engine.prefill(prompt, blocks, chunk=32)  # 5 chunks, the last one ragged
    ops.read_status(engine._prefill_attn_ws, "prefill attention")
    ops.read_status(engine._prefill_moe_ws, "prefill moe")
    assert rel_err(logits_b, logits_a) < TOL_MODEL and first_a == first_b
    for a, p in zip(k_a, engine.k_pools):
        assert rel_err(p[blocks], a) < TOL_MODEL  # same pages written either way
    # prefix hit: the first 64 tokens (4 full pages) are already in the pages; only the suffix is run
    first_c, logits_c = engine.prefill(prompt, blocks, cached_tokens=64, chunk=256)
    assert rel_err(logits_c, logits_a) < TOL_MODEL and first_c == first_a


def test_prefill_then_decode_matches_prefill_of_the_longer_prompt(ops):
    """Decoding token t after a prompt gives the logits that a prompt pass over prompt + [t] gives."""
    engine = make_engine()
    backend = pkg("backend").B200Backend(engine, max_new_tokens=16)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 4096, (45,), generator=g).tolist()
    kv, first, n = backend.prefill(prompt, "s")
    batch = backend.splice_into_batched(None, kv, n)
    nxt, batch = backend.decode_step_batched(torch.tensor([[first]]), batch, None, None)
    dec_logits = engine.last_logits[0].clone()
    tok2, logits2 = engine.prefill(prompt + [first], list(range(40, 48)))
    assert rel_err(dec_logits, logits2) < TOL_MODEL
    assert int(nxt[0]) == tok2 or float(torch.topk(logits2.float(), 2).values.diff().abs()) < 0.05


def test_merged_decode_step_and_prompt_chunk_equals_the_two_passes(ops):
    """One pass over the model for the decode rows and a prompt chunk of another sequence gives what the
    chunk's pass followed by the decode step gives: tokens, the chunk's pages, the decode rows' new K/V and
    the logits of the step after (which reads everything the merged pass wrote)."""
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (37, 90)]
    new = torch.randint(0, 4096, (75,), generator=g).tolist()
    forced = [torch.randint(0, 4096, (2,), generator=g) for _ in range(3)] + [torch.randint(0, 4096, (3,), generator=g)]

    def serve(merged):
        engine = make_engine()
        backend = pkg("backend").B200Backend(engine, max_new_tokens=16)
        batch = None
        for i, p in enumerate(prompts):
            kv, first, n = backend.prefill(p, f"s{i}")
            batch = backend.splice_into_batched(batch, kv, n)
        partial, trace = None, []
        for step, lo in enumerate(range(0, len(new), 32)):  # chunks of 32, 32 and 11 tokens
            piece = new[lo:lo + 32]
            tok = forced[step].view(-1, 1)  # the same input tokens either way, whatever the step before gave
            if merged:
                nxt, batch, partial, last, n = backend.decode_step_with_prefill_chunk(tok, batch, piece, partial)
            else:
                partial, last, n = backend.prefill_chunk(piece, partial)
                nxt, batch = backend.decode_step_batched(tok, batch, None, None)
            trace.append((nxt.tolist(), last, n))
        # the new sequence joins the batch; one more step reads every page written above
        batch = backend.splice_into_batched(batch, partial, partial.ctx_len)
        nxt, batch = backend.decode_step_batched(forced[3].view(-1, 1), batch, None, None)
        engine.check_status("merged pass test")
        pages = partial.block_ids[: (len(new) + 15) // 16]
        return trace, nxt.tolist(), engine.last_logits.float().clone(), [p[pages].float().clone() for p in engine.k_pools], \
            [p[pages].float().clone() for p in engine.v_pools], partial.block_ids

    tr_a, nxt_a, logits_a, k_a, v_a, ids_a = serve(False)
    tr_b, nxt_b, logits_b, k_b, v_b, ids_b = serve(True)
    assert ids_a == ids_b and [t[2] for t in tr_a] == [t[2] for t in tr_b]
    for a, b in zip(k_a + v_a, k_b + v_b):
        assert rel_err(b, a) < TOL_MODEL
    assert rel_err(logits_b, logits_a) < TOL_MODEL
    # tokens: equal wherever the two-pass logits decide clearly (the merged pass has other GEMM shapes, i.e.
    # other bf16 rounding points, as with any re-chunking above)
    top2 = torch.topk(logits_a, 2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.05
    for i in range(len(nxt_a)):
        assert nxt_a[i] == nxt_b[i] or not bool(clear[i])
    flat_a = [t for a in tr_a for t in a[0] + [a[1]]]
    flat_b = [t for b in tr_b for t in b[0] + [b[1]]]
    assert sum(x == y for x, y in zip(flat_a, flat_b)) >= len(flat_a) - 2, (tr_a, tr_b)  # 9 tokens, near-ties aside
