"""Oracle: RMSNorm, rotary embedding and the page write on CPU (test infrastructure only)."""
from __future__ import annotations

import torch


def rms_norm_ref(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """transformers ``Qwen3MoeRMSNorm.forward``: statistics in fp32, the normalised value cast back
    to the input dtype, then multiplied by the weight."""
    dt = x.dtype
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    return weight * (xf * torch.rsqrt(var + eps)).to(dt)


def rope_tables_ref(head_dim: int, theta: float, max_pos: int, dtype=torch.bfloat16):
    """transformers rotary embedding, default type: inv_freq = theta^(-2i/d); cos/sin of
    cat(freqs, freqs), computed in fp32 and cast to the model dtype."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rope_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """transformers ``apply_rotary_pos_emb`` / ``rotate_half`` on fp32 values:
    x * cos + cat(-x2, x1) * sin with x1, x2 the two halves of the last axis."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x.float() * cos.float() + rot.float() * sin.float()


def qk_norm_rope_append_ref(qkv, q_w, k_w, cos, sin, positions, block_table, k_pool, v_pool, hq, eps):
    """What the attention module does before the attention product for one new token per row
    (transformers ``Qwen3MoeAttention.forward``: q_norm/k_norm on the head axis, rotary embedding,
    cache update), with the cache update expressed as a page-slot write in the reference pool
    layout (src/inference_server/kv_cache/block_manager.py:33-49).  Returns q [B, Hq, D] fp32 and
    updates copies of the pools."""
    B, heads, D = qkv.shape
    hkv = k_pool.shape[1]
    page = k_pool.shape[2]
    k_pool, v_pool = k_pool.clone(), v_pool.clone()
    q = rms_norm_ref(qkv[:, :hq], q_w, eps)
    k = rms_norm_ref(qkv[:, hq:hq + hkv], k_w, eps)
    v = qkv[:, hq + hkv:]
    c = cos[positions.long()].unsqueeze(1)
    s = sin[positions.long()].unsqueeze(1)
    q = apply_rope_ref(q, c, s)
    k = apply_rope_ref(k, c, s)
    for b in range(B):
        pos = int(positions[b])
        bid = int(block_table[b, pos // page])
        k_pool[bid, :, pos % page, :] = k[b].to(k_pool.dtype)
        v_pool[bid, :, pos % page, :] = v[b]
    return q, k_pool, v_pool
