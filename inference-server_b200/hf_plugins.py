"""The kernels as plug-ins of the HuggingFace model forward the reference already runs.

``TorchBackend.decode_step_batched`` (src/inference_server/backends/torch_backend.py:305-322) calls
``self.model(input_ids, attention_mask=..., position_ids=..., past_key_values=..., use_cache=True)``.  Inside,
a Qwen3-MoE model looks its attention function up by ``config._attn_implementation`` and its experts function
by ``config._experts_implementation``, and grows the KV cache through ``past_key_values.update``.  This module
registers one implementation for each hook, so that the unchanged model forward runs on this package's kernels:

  ``"b200_paged"``  attention: one query token per row over the KV page pools (``b200_paged_attn_decode``)
  ``"b200_fp8"``    experts: e4m3 128x128-block weights, grouped tcgen05 GEMMs (quantised once per module)
  ``PagedKVCache``  a ``Cache`` whose ``update`` writes the step's K/V rows into their page slots
                    (``b200_kv_append``) instead of concatenating

The attention hook needs the block table, so the cache object is also passed to the model call as the keyword
``b200_cache`` (extra keywords reach the attention function untouched).  Decode steps (one new token per row)
only; prompts go through ``DecodeEngine.prefill``.
"""
from __future__ import annotations

import torch
from transformers.cache_utils import Cache, CacheLayerMixin

from . import ops, quant

PAGE = 16


class _PagedLayer(CacheLayerMixin):
    """Layer view of the page pools: `update` appends one token per row."""

    is_sliding = False

    def __init__(self, cache: "PagedKVCache", layer_idx: int):
        super().__init__()
        self.cache, self.layer_idx = cache, layer_idx
        self.is_initialized = True

    def lazy_initialization(self, key_states, value_states) -> None:
        pass

    def update(self, key_states, value_states, *args, **kwargs):
        c = self.cache
        if key_states.shape[2] != 1:
            raise ValueError("PagedKVCache takes one new token per row (decode steps)")
        ops.kv_append(key_states[:, :, 0, :].contiguous(), value_states[:, :, 0, :].contiguous(),
                      c.k_pools[self.layer_idx], c.v_pools[self.layer_idx], c.block_table, c.positions, c.status)
        return key_states, value_states

    def get_seq_length(self) -> int:
        return self.cache.max_len

    def get_mask_sizes(self, query_length: int) -> tuple[int, int]:
        return self.cache.max_len + query_length, 0

    def get_max_cache_shape(self) -> int:
        return -1


class PagedKVCache(Cache):
    """KV cache over page pools in the reference layout [num_blocks, kv_heads, 16, head_dim] per layer
    (src/inference_server/kv_cache/block_manager.py:33-49).

    block_table [B, max_pages] int32, positions [B] int32 = tokens already stored per row (the index the next
    token is written at).  Call ``advance()`` after each model forward."""

    def __init__(self, k_pools, v_pools, block_table: torch.Tensor, positions: torch.Tensor,
                 split_tokens: int | None = None):
        self.k_pools, self.v_pools = k_pools, v_pools
        self.block_table, self.positions = block_table, positions
        self.status = torch.zeros(64, dtype=torch.int32, device=block_table.device)
        self.max_len = int(positions.max().item()) if positions.numel() else 0
        B, hkv = block_table.shape[0], k_pools[0].shape[1]
        self.split_tokens = split_tokens or ops.default_split_tokens(B, hkv, block_table.shape[1] * PAGE)
        self._ws = None
        super().__init__(layers=[_PagedLayer(self, i) for i in range(len(k_pools))])

    def workspace(self, num_q_heads: int, head_dim: int) -> torch.Tensor:
        if self._ws is None:
            self._ws = ops.paged_attn_workspace(self.block_table.shape[0], num_q_heads, head_dim,
                                                self.block_table.shape[1], PAGE, self.split_tokens,
                                                self.block_table.device)
        return self._ws

    def advance(self) -> None:
        self.positions += 1
        self.max_len += 1


def paged_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0, scaling: float | None = None,
                            sliding_window=None, b200_cache: PagedKVCache | None = None, **kwargs):
    """Attention hook: query [B, Hq, 1, D]; `key`/`value` are this step's rows only (already written to their
    page slots by ``PagedKVCache.update``); the mask is ignored - context lengths come from the cache."""
    if b200_cache is None:
        raise ValueError("pass the PagedKVCache to the model call as b200_cache=...")
    B, Hq, Sq, D = query.shape
    if Sq != 1:
        raise ValueError("b200_paged attention handles decode steps (one query token per row)")
    li = module.layer_idx
    out = ops.paged_attn_decode(query[:, :, 0, :].contiguous(), b200_cache.k_pools[li], b200_cache.v_pools[li],
                                b200_cache.block_table, b200_cache.positions + 1,
                                scaling if scaling is not None else D ** -0.5, b200_cache.split_tokens,
                                b200_cache.workspace(Hq, D))
    return out.view(B, 1, Hq, D), None


def fp8_experts_forward(self, hidden_states, top_k_index, top_k_weights):
    """Experts hook: (experts module, hidden [T, H], ids [T, K], weights [T, K]) -> [T, H].  The module's
    ``gate_up_proj`` [E, 2I, H] and ``down_proj`` [E, H, I] are quantised to e4m3 128x128 blocks on first use."""
    w = getattr(self, "_b200_fp8", None)
    if w is None:
        w13, w13s = quant.quantize_weight_blocks(self.gate_up_proj.detach().float())
        w2, w2s = quant.quantize_weight_blocks(self.down_proj.detach().float())
        w = (quant.tile_weight_blocks(w13), w13s, quant.tile_weight_blocks(w2), w2s)
        self._b200_fp8 = w
    x = hidden_states.to(torch.bfloat16).contiguous()
    ids = top_k_index.to(torch.int32).contiguous()
    perm, xq, xs = ops.moe_permute_quant(ids, x, self.num_experts)
    hq, hs = ops.moe_fp8_gemm_gate_up(xq, xs, w[0], w[1], perm)
    y = ops.moe_fp8_gemm_down(hq, hs, w[2], w[3], perm)
    return ops.moe_combine(y, perm.row_of_pair, top_k_weights.float().contiguous()).to(hidden_states.dtype)


def register() -> None:
    """Register both hooks with transformers (idempotent)."""
    from transformers import AttentionInterface
    from transformers.integrations.moe import ExpertsInterface

    AttentionInterface.register("b200_paged", paged_attention_forward)
    ExpertsInterface.register("b200_fp8", fp8_experts_forward)
