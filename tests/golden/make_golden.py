"""Generates the golden fixtures in this directory from the REAL reference.

Run where the reference checkout exists (default: a directory `reference` next to this
repository; override with REFERENCE_ROOT):

    python tests/golden/make_golden.py

It imports the reference's own kv_cache / backend code and the installed
``transformers`` Qwen3-MoE modules (the arithmetic the reference calls into),
runs them on seeded inputs and stores inputs + outputs as small .npz files.
The GPU box has no reference checkout, so tests read only these files.
"""
from __future__ import annotations

import os
import random
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("REFERENCE_ROOT", os.path.join(os.path.dirname(REPO), "reference"))
sys.path.insert(0, os.path.join(REF, "src"))

from inference_server.kv_cache.block_manager import BlockManager  # noqa: E402
from inference_server.kv_cache.cache_manager import CacheManager  # noqa: E402
from inference_server.kv_cache.hf_format import blocks_to_dynamic_cache  # noqa: E402
from inference_server.backends.torch_backend import TorchBackend  # noqa: E402
from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM  # noqa: E402
from transformers.models.qwen3_moe import modeling_qwen3_moe as hfm  # noqa: E402
from transformers.integrations.finegrained_fp8 import Fp8Dequantize, Fp8Quantize  # noqa: E402


def save(name, **arrays):
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **arrays)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def attention_case(name, hq, hkv, d, page, ctx_lens, share_first_pages, seed):
    """Pools and gather by the reference's BlockManager / blocks_to_dynamic_cache;
    attention by transformers eager_attention_forward."""
    g = torch.Generator().manual_seed(seed)
    n_pages = [(L + page - 1) // page for L in ctx_lens]
    num_blocks = sum(n_pages) + 3
    bm = BlockManager(num_blocks, page, layer_shapes=[(hkv, d)], device="cpu", dtype=torch.float32)
    bm.k_pools[0].copy_(torch.randn(bm.k_pools[0].shape, generator=g))
    bm.v_pools[0].copy_(torch.randn(bm.v_pools[0].shape, generator=g))
    rng = random.Random(seed)
    free = list(range(num_blocks))
    rng.shuffle(free)
    shared = [free.pop() for _ in range(share_first_pages)]
    B = len(ctx_lens)
    table = np.zeros((B, max(n_pages)), dtype=np.int32)
    q = torch.randn(B, hq, d, generator=g)
    out = np.zeros((B, hq, d), dtype=np.float32)
    module = types.SimpleNamespace(num_key_value_groups=hq // hkv, training=False)
    for b, L in enumerate(ctx_lens):
        ids = []
        for p in range(n_pages[b]):
            full = (p + 1) * page <= L
            ids.append(shared[p] if (p < share_first_pages and full) else free.pop())
        table[b, : len(ids)] = ids
        blocks = []
        left = L
        for bid in ids:
            blk = bm.get_block(bid)
            blk.token_ids = list(range(min(page, left)))  # only the count matters
            left -= page
            blocks.append(blk)
        cache, n = blocks_to_dynamic_cache(blocks)
        assert n == L
        k, v = cache.layers[0].keys, cache.layers[0].values  # [1, Hkv, L, D]
        o, _ = hfm.eager_attention_forward(module, q[b].view(1, hq, 1, d), k, v, None, scaling=d ** -0.5)
        out[b] = o.view(hq, d).numpy()  # o is [1, 1, Hq, D]
    save(name, q=q.numpy(), k_pool=bm.k_pools[0].numpy(), v_pool=bm.v_pools[0].numpy(), block_table=table,
         ctx_lens=np.array(ctx_lens, dtype=np.int32), out=out, scale=np.float32(d ** -0.5))


def prefill_attention_case(name, hq, hkv, d, page, prefix, chunk, seed):
    """A prompt suffix of `chunk` tokens on top of `prefix` cached tokens: pools and gather by the reference's
    BlockManager / blocks_to_dynamic_cache, attention by transformers eager_attention_forward with the additive
    causal mask the model builds for a suffix (row of position p sees tokens 0..p)."""
    g = torch.Generator().manual_seed(seed)
    L = prefix + chunk
    n_pages = (L + page - 1) // page
    bm = BlockManager(n_pages + 5, page, layer_shapes=[(hkv, d)], device="cpu", dtype=torch.float32)
    bm.k_pools[0].copy_(torch.randn(bm.k_pools[0].shape, generator=g))
    bm.v_pools[0].copy_(torch.randn(bm.v_pools[0].shape, generator=g))
    ids = list(range(n_pages + 5))
    random.Random(seed).shuffle(ids)
    ids = ids[:n_pages]
    blocks, left = [], L
    for bid in ids:
        blk = bm.get_block(bid)
        blk.token_ids = list(range(min(page, left)))  # only the count matters
        left -= page
        blocks.append(blk)
    cache, n = blocks_to_dynamic_cache(blocks)
    assert n == L
    k, v = cache.layers[0].keys, cache.layers[0].values  # [1, Hkv, L, D]
    q = torch.randn(chunk, hq, d, generator=g)
    pos = prefix + torch.arange(chunk)
    mask = torch.where(torch.arange(L).view(1, L) <= pos.view(chunk, 1), 0.0, float("-inf")).view(1, 1, chunk, L)
    module = types.SimpleNamespace(num_key_value_groups=hq // hkv, training=False)
    o, _ = hfm.eager_attention_forward(module, q.permute(1, 0, 2).unsqueeze(0), k, v, mask, scaling=d ** -0.5)
    save(name, q=q.numpy(), k_pool=bm.k_pools[0].numpy(), v_pool=bm.v_pools[0].numpy(),
         table_row=np.array(ids, dtype=np.int32), first_pos=np.int32(prefix), out=o[0].numpy(),
         scale=np.float32(d ** -0.5))


def router_case(name, T, H, E, K, seed):
    torch.manual_seed(seed)
    cfg = types.SimpleNamespace(num_experts_per_tok=K, num_experts=E, norm_topk_prob=True, hidden_size=H)
    router = hfm.Qwen3MoeTopKRouter(cfg)
    with torch.no_grad():
        router.weight.copy_(torch.randn(E, H) * 0.5)
        x = torch.randn(T, H)
        logits = torch.nn.functional.linear(x, router.weight)
        _, scores, idx = router(x)
    save(name, logits=logits.numpy(), topk_ids=idx.numpy().astype(np.int32), topk_weights=scores.numpy())


def experts_case(name, T, H, I, E, K, seed):
    torch.manual_seed(seed)
    cfg = types.SimpleNamespace(num_experts=E, hidden_size=H, moe_intermediate_size=I, hidden_act="silu",
                                num_experts_per_tok=K, norm_topk_prob=True)
    experts = hfm.Qwen3MoeExperts(cfg)
    router = hfm.Qwen3MoeTopKRouter(cfg)
    with torch.no_grad():
        experts.gate_up_proj.copy_(torch.randn(E, 2 * I, H) * 0.1)
        experts.down_proj.copy_(torch.randn(E, H, I) * 0.1)
        router.weight.copy_(torch.randn(E, H) * 0.5)
        x = torch.randn(T, H)
        logits = torch.nn.functional.linear(x, router.weight)
        _, scores, idx = router(x)
        out = hfm.Qwen3MoeExperts.forward.__wrapped__(experts, x, idx, scores) if hasattr(
            hfm.Qwen3MoeExperts.forward, "__wrapped__") else None
        if out is None:
            experts.config = types.SimpleNamespace(_experts_implementation="eager")
            out = experts(x, idx, scores)
    save(name, x=x.numpy(), logits=logits.numpy(), gate_up_proj=experts.gate_up_proj.detach().numpy(),
         down_proj=experts.down_proj.detach().numpy(), out=out.numpy(), top_k=np.int32(K))


def weight_quant_case(name, seed):
    torch.manual_seed(seed)
    w = torch.randn(2, 128, 256) * 0.02
    w[1, :, :128] = 0.0  # an all-zero tile exercises the amax == 0 rule
    qcfg = types.SimpleNamespace(weight_block_size=(128, 128))
    op = Fp8Quantize(types.SimpleNamespace(quantization_config=qcfg))
    res = op.convert({"experts.gate_up_proj": [w]})
    q = res["experts.gate_up_proj"]
    s = res["experts.gate_up_proj_scale_inv"]
    save(name, w=w.numpy(), q=q.view(torch.uint8).numpy(), scale_inv=s.numpy())


def weight_dequant_case(name, seed):
    """transformers Fp8Dequantize.convert on a 2 x 3 grid of 128x128 tiles with six different scales: pins
    which axis of scale_inv follows the rows and which the columns of the weight, and that w = q * scale_inv."""
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 256, (1, 256, 384), generator=g, dtype=torch.int32)
    codes = torch.where((codes & 0x7F) == 0x7F, codes & 0x80, codes).to(torch.uint8)  # no NaN encodings
    q = codes.view(torch.float8_e4m3fn)
    scale_inv = (torch.rand(1, 2, 3, generator=g) * 0.01 + 1e-4).float()
    qcfg = types.SimpleNamespace(weight_block_size=(128, 128))
    op = Fp8Dequantize(types.SimpleNamespace(quantization_config=qcfg))
    out = op.convert({"weight$": [q], "weight_scale_inv": [scale_inv]}, full_layer_name="w")["w"]
    save(name, q=codes.numpy(), scale_inv=scale_inv.numpy(), w=out.float().numpy())


def tiny_model_config():
    return Qwen3MoeConfig(
        vocab_size=4096, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
        num_attention_heads=8, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
        rope_theta=1e6, rope_parameters={"rope_type": "default", "rope_theta": 1e6},
        num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256, norm_topk_prob=True,
        decoder_sparse_step=1, mlp_only_layers=[], max_position_embeddings=4096,
        tie_word_embeddings=False, attn_implementation="eager", experts_implementation="eager",
        initializer_range=0.02,
    )


def tiny_model_case(name):
    """Config 1: 4 prompts, 32 greedy steps through the reference's TorchBackend
    primitives, driven the way ContinuousBatchScheduler does
    (src/inference_server/scheduler.py:355-402)."""
    torch.manual_seed(0)
    model = Qwen3MoeForCausalLM(tiny_model_config()).float().eval()
    backend = TorchBackend(device="cpu")
    backend.model = model
    backend._eos_ids = set()
    shapes = backend.kv_shape_per_layer()
    cache = CacheManager(256, 16, layer_shapes=shapes, device="cpu", dtype=torch.float32)
    backend.set_cache_adapter(cache)
    rng = random.Random(0)
    prompts = [[rng.randrange(4096) for _ in range(rng.randint(32, 128))] for _ in range(4)]
    batched, mask, cur, lens = None, None, [], []
    for p in prompts:
        kv, first, n = backend.prefill(p, "s")
        if batched is None:
            batched = backend.splice_into_batched(None, kv, n)
            mask = torch.ones(1, n, dtype=torch.long)
        else:
            ex = backend.kv_length(batched)
            mx = max(ex, n)
            batched = backend.splice_into_batched(batched, kv, n)
            if mx > ex:
                mask = torch.cat([torch.zeros(mask.shape[0], mx - ex, dtype=torch.long), mask], dim=1)
            row = torch.zeros(1, mx, dtype=torch.long)
            row[0, mx - n:] = 1
            mask = torch.cat([mask, row], dim=0)
        cur.append(first)
        lens.append(n)
    steps = 32
    tokens = np.zeros((steps + 1, 4), dtype=np.int64)
    tokens[0] = cur
    top2 = np.zeros((steps, 4, 2), dtype=np.float32)
    keep = {0: None, 15: None, 31: None}
    for s in range(steps):
        ct = torch.tensor([[t] for t in cur])
        mask = torch.cat([mask, torch.ones(4, 1, dtype=torch.long)], dim=1)
        pos = torch.tensor([[n] for n in lens])
        with torch.no_grad():
            outputs = model(ct, attention_mask=mask, position_ids=pos, past_key_values=batched, use_cache=True)
        logits = outputs.logits[:, -1, :]
        nxt = logits.argmax(dim=-1)
        # the same call through the reference entry point must agree (it re-runs the forward on a
        # cache that already grew, so it is only used for the first step's cross-check)
        top2[s] = torch.topk(logits, 2, dim=-1).values.numpy()
        if s in keep:
            keep[s] = logits.numpy().copy()
        batched = outputs.past_key_values
        cur = [int(t) for t in nxt]
        lens = [n + 1 for n in lens]
        tokens[s + 1] = cur
    flat = np.concatenate([np.array(p, dtype=np.int64) for p in prompts])
    save(name, prompt_flat=flat, prompt_lens=np.array([len(p) for p in prompts], dtype=np.int64),
         tokens=tokens, top2=top2, logits_step0=keep[0], logits_step15=keep[15], logits_step31=keep[31])


def tiny_model_backend_crosscheck():
    """decode_step_batched (torch_backend.py:305-322) on the same state gives the same first token
    as the direct forward above; run separately so its cache growth does not disturb the loop."""
    torch.manual_seed(0)
    model = Qwen3MoeForCausalLM(tiny_model_config()).float().eval()
    backend = TorchBackend(device="cpu")
    backend.model = model
    backend._eos_ids = set()
    rng = random.Random(0)
    p = [rng.randrange(4096) for _ in range(rng.randint(32, 128))]
    kv, first, n = backend.prefill(p, "s")
    batched = backend.splice_into_batched(None, kv, n)
    mask = torch.ones(1, n + 1, dtype=torch.long)
    nxt, _ = backend.decode_step_batched(torch.tensor([[first]]), batched, mask, torch.tensor([[n]]))
    return int(first), int(nxt[0])


if __name__ == "__main__":
    only = set(sys.argv[1:])  # file names to (re)generate; none given = all
    if only:
        if "fp8_weight_dequant.npz" in only:
            weight_dequant_case("fp8_weight_dequant.npz", seed=8)
        if "attn_prefill_d64.npz" in only:
            prefill_attention_case("attn_prefill_d64.npz", hq=8, hkv=2, d=64, page=16, prefix=37, chunk=45, seed=9)
        if only - {"fp8_weight_dequant.npz", "attn_prefill_d64.npz"}:
            raise SystemExit("selective generation is offered for the two newest fixtures only; run without arguments")
        sys.exit(0)
    attention_case("attn_d64.npz", hq=8, hkv=2, d=64, page=16, ctx_lens=[1, 16, 17, 95, 130, 64],
                   share_first_pages=3, seed=1)
    attention_case("attn_d128.npz", hq=16, hkv=2, d=128, page=16, ctx_lens=[150, 33, 129],
                   share_first_pages=2, seed=2)
    prefill_attention_case("attn_prefill_d64.npz", hq=8, hkv=2, d=64, page=16, prefix=37, chunk=45, seed=9)
    router_case("route_e128k8.npz", T=96, H=64, E=128, K=8, seed=3)
    router_case("route_e16k4.npz", T=64, H=32, E=16, K=4, seed=4)
    experts_case("experts_dense.npz", T=24, H=64, I=32, E=8, K=2, seed=5)
    weight_quant_case("fp8_weight_quant.npz", seed=6)
    weight_dequant_case("fp8_weight_dequant.npz", seed=8)
    tiny_model_case("c1_tiny.npz")
    print("backend cross-check (first, next):", tiny_model_backend_crosscheck())
