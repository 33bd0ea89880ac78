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
