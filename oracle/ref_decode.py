"""Oracle / CPU baseline: the reference's decode step on host cores (test infrastructure only).

Restates ``TorchBackend.decode_step_batched``
(src/inference_server/backends/torch_backend.py:305-322) and the state the
scheduler keeps around it (src/inference_server/scheduler.py:379-402): a dense,
left-padded HuggingFace ``DynamicCache`` [B, Hkv, S, D], an int64 attention mask
that grows by one column per step, explicit ``position_ids``, one model forward
and an argmax.  The arithmetic is the installed ``transformers`` Qwen3-MoE model,
which is exactly what the reference calls.

The reference checkout cannot travel to the benchmark machine, so this file is a
restatement ("port"); tests/golden/c1_tiny.npz pins it against tokens produced by
the reference's own TorchBackend.
"""
from __future__ import annotations

import time

import torch


def hf_config(cfg, num_layers: int | None = None, **extra):
    """transformers Qwen3MoeConfig for one of the engine's ModelConfig shapes."""
    from transformers import Qwen3MoeConfig

    return Qwen3MoeConfig(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden, intermediate_size=4 * cfg.hidden,
        num_hidden_layers=num_layers or cfg.layers, num_attention_heads=cfg.q_heads,
        num_key_value_heads=cfg.kv_heads, head_dim=cfg.head_dim, rms_norm_eps=cfg.rms_eps,
        rope_theta=cfg.rope_theta, rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_theta},
        num_experts=cfg.experts, num_experts_per_tok=cfg.top_k, moe_intermediate_size=cfg.moe_inter,
        norm_topk_prob=cfg.norm_topk_prob, decoder_sparse_step=1, mlp_only_layers=[],
        max_position_embeddings=40960, tie_word_embeddings=False, initializer_range=0.02, **extra)


def decode_step_batched(model, current_tokens, batched_kv, attention_mask, position_ids):
    """torch_backend.py:305-322, verbatim in behaviour."""
    with torch.no_grad():
        outputs = model(current_tokens, attention_mask=attention_mask, position_ids=position_ids,
                        past_key_values=batched_kv, use_cache=True)
    return outputs.logits[:, -1, :].argmax(dim=-1), outputs.past_key_values


def dense_left_padded_cache(num_layers, ctx_lens, kv_heads, head_dim, dtype, seed=0):
    """A batched DynamicCache as ``_stack_caches_left_padded`` builds it
    (torch_backend.py:237-258): rows right-aligned, zeros on the left; contents N(0,1)."""
    from transformers.cache_utils import DynamicCache

    g = torch.Generator().manual_seed(seed)
    B, S = len(ctx_lens), max(ctx_lens)
    cache = DynamicCache()
    mask = torch.zeros(B, S, dtype=torch.long)
    for i, L in enumerate(ctx_lens):
        mask[i, S - L:] = 1
    for layer in range(num_layers):
        k = torch.randn(B, kv_heads, S, head_dim, generator=g).to(dtype)
        v = torch.randn(B, kv_heads, S, head_dim, generator=g).to(dtype)
        keep = mask.view(B, 1, S, 1).to(dtype)
        cache.update(k * keep, v * keep, layer)
    return cache, mask


def time_reference_decode(cfg, ctx_lens, steps: int, warmup: int, sample_layers: int = 1,
                          dtype=torch.bfloat16, seed: int = 0, budget_s: float | None = None) -> dict:
    """Times the reference decode step on the host for `sample_layers` of cfg.layers
    layers at the full batch and extrapolates the layer part to the full depth.
    With `budget_s` the loop stops early (after at least one timed step) once that many
    seconds of stepping have gone by; `steps_done` and `warmup_done` say what ran.

    Returns dict(step_s_sample, layer_s, other_s, step_s_full, tok_per_s, threads, sample,
    steps_done, warmup_done, stepping_s)."""
    from transformers import Qwen3MoeForCausalLM

    torch.manual_seed(seed)
    model = Qwen3MoeForCausalLM(hf_config(cfg, sample_layers)).to(dtype).eval()
    B = len(ctx_lens)
    cache, mask = dense_left_padded_cache(sample_layers, ctx_lens, cfg.kv_heads, cfg.head_dim, dtype, seed)
    layer_time = [0.0]

    def pre(_m, _a, _k=None):
        layer_time.append(time.perf_counter())

    def post(_m, _a, _o):
        layer_time[0] += time.perf_counter() - layer_time.pop()

    handles = []
    for lyr in model.model.layers:
        handles.append(lyr.register_forward_pre_hook(pre))
        handles.append(lyr.register_forward_hook(post))
    cur = torch.randint(0, cfg.vocab_size, (B, 1), generator=torch.Generator().manual_seed(seed))
    lens = list(ctx_lens)
    step_times, layer_times = [], []
    t_loop = time.perf_counter()
    warmup_done = 0
    for s in range(warmup + steps):
        if budget_s is not None and time.perf_counter() - t_loop > budget_s and (step_times or s >= 1):
            if step_times:
                break
            warmup = s  # the budget went into warm-up steps: time one step now and stop
        warmup_done = min(s, warmup)
        mask = torch.cat([mask, torch.ones(B, 1, dtype=torch.long)], dim=1)  # scheduler.py:386-389
        pos = torch.tensor([[n] for n in lens])                              # scheduler.py:390-393
        layer_time[0] = 0.0
        t0 = time.perf_counter()
        nxt, cache = decode_step_batched(model, cur, cache, mask, pos)
        dt = time.perf_counter() - t0
        cur = nxt.view(B, 1)
        lens = [n + 1 for n in lens]
        if s >= warmup:
            step_times.append(dt)
            layer_times.append(layer_time[0] / sample_layers)
            warmup_done = warmup
    stepping_s = time.perf_counter() - t_loop
    steps = len(step_times)
    for h in handles:
        h.remove()
    step_s = sum(step_times) / len(step_times)
    layer_s = sum(layer_times) / len(layer_times)
    other_s = max(step_s - layer_s * sample_layers, 0.0)
    full = other_s + layer_s * cfg.layers
    return dict(step_s_sample=step_s, layer_s=layer_s, other_s=other_s, step_s_full=full, tok_per_s=B / full,
                threads=torch.get_num_threads(), steps_done=steps, warmup_done=warmup_done, stepping_s=stepping_s,
                sample=f"{sample_layers} of {cfg.layers} layers at the full batch of {B} rows (dense left-padded "
                       f"{str(dtype).replace('torch.', '')} cache, S={max(ctx_lens)}), {steps} steps; step time = "
                       f"embed+norm+lm_head+argmax time + {cfg.layers} x measured layer time")
