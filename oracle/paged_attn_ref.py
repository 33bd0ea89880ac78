"""Oracle: paged GQA decode attention on CPU (test infrastructure only)."""
from __future__ import annotations

import torch


def gather_pages(pool: torch.Tensor, block_ids, ctx_len: int) -> torch.Tensor:
    """Dense [Hkv, ctx_len, D] view of one sequence.

    Follows ``blocks_to_dynamic_cache`` (src/inference_server/kv_cache/hf_format.py:21-45):
    per block the slice ``pool[block_id, :, :n, :]`` (``Block.k_tensor``,
    kv_cache/block.py:34-41) concatenated on the sequence axis; every page is
    full except the last.  Pool layout [num_blocks, Hkv, page, D] is
    kv_cache/block_manager.py:33-49.
    """
    page = pool.shape[2]
    parts = []
    left = ctx_len
    for bid in block_ids:
        if left <= 0:
            break
        n = min(page, left)
        parts.append(pool[int(bid), :, :n, :])
        left -= n
    if not parts:
        return pool.new_zeros(pool.shape[1], 0, pool.shape[3])
    return torch.cat(parts, dim=1)


def paged_attn_ref(q, k_pool, v_pool, block_table, ctx_lens, scale: float) -> torch.Tensor:
    """softmax(q K^T * scale) V per row, fp32 arithmetic, output fp32 [B, Hq, D].

    Follows the eager attention formula the reference's model forward uses
    (transformers qwen3_moe ``eager_attention_forward``: repeat_kv, matmul,
    softmax in fp32, matmul) for one query token per row with no mask (every
    gathered key is visible to the newest token).
    """
    q = q.detach().cpu()
    k_pool, v_pool = k_pool.detach().cpu(), v_pool.detach().cpu()
    B, Hq, D = q.shape
    Hkv = k_pool.shape[1]
    rep = Hq // Hkv
    out = torch.zeros(B, Hq, D, dtype=torch.float32)
    for b in range(B):
        L = int(ctx_lens[b])
        if L == 0:
            continue
        k = gather_pages(k_pool, block_table[b].tolist(), L).float()  # [Hkv, L, D]
        v = gather_pages(v_pool, block_table[b].tolist(), L).float()
        k = k.repeat_interleave(rep, dim=0)  # [Hq, L, D]
        v = v.repeat_interleave(rep, dim=0)
        s = torch.einsum("hd,hld->hl", q[b].float(), k) * scale
        p = torch.softmax(s, dim=-1, dtype=torch.float32)
        out[b] = torch.einsum("hl,hld->hd", p, v)
    return out


def paged_prefill_ref(q, k_pool, v_pool, table_row, first_pos: int, scale: float) -> torch.Tensor:
    """Causal attention of a chunk of R consecutive prompt tokens (positions first_pos ..) over the pages of
    their sequence, fp32, output [R, Hq, D].

    This is what the reference computes for a prompt suffix on top of a cached prefix: the prefix pages are
    gathered into a dense cache (``blocks_to_dynamic_cache``, src/inference_server/kv_cache/hf_format.py:21-45)
    and the suffix runs through the model with a causal mask
    (src/inference_server/backends/torch_backend.py:107-147 -> transformers ``eager_attention_forward`` with the
    additive causal mask: token t is visible to the row of position p iff t <= p).  The K/V of the chunk itself
    are expected in their page slots already.
    """
    q = q.detach().cpu().float()
    R, Hq, D = q.shape
    Hkv = k_pool.shape[1]
    rep = Hq // Hkv
    L = first_pos + R
    ids = [int(b) for b in table_row]
    k = gather_pages(k_pool.detach().cpu(), ids, L).float().repeat_interleave(rep, dim=0)  # [Hq, L, D]
    v = gather_pages(v_pool.detach().cpu(), ids, L).float().repeat_interleave(rep, dim=0)
    s = torch.einsum("rhd,hld->hrl", q, k) * scale
    visible = torch.arange(L).view(1, 1, L) <= (first_pos + torch.arange(R)).view(1, R, 1)
    s = s.masked_fill(~visible, float("-inf"))
    p = torch.softmax(s, dim=-1, dtype=torch.float32)
    return torch.einsum("hrl,hld->rhd", p, v).contiguous()
