"""Operator wrappers: torch CUDA tensors in, C-ABI calls out.

Each function checks shapes/dtypes/contiguity, passes raw device pointers and
the current torch CUDA stream to ``libb200decode.so`` and returns torch tensors.
Nothing here computes on the host and nothing falls back to torch ops: without
the library, or off a CUDA device, the calls raise.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check

DTYPE_CODE = {torch.bfloat16: 0, torch.float32: 1}


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, name: str, dtype=None):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this path has no CPU implementation)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")


def read_status(status: torch.Tensor, where: str = "device status") -> None:
    """Synchronise and raise if the device status word at the start of `status` is set."""
    rc = _lib.load().b200_read_status(status.data_ptr(), _stream())
    check(rc, where)


# ------------------------------------------------------------ paged attention


def default_split_tokens(batch: int, num_kv_heads: int, max_ctx: int, num_sms: int = 148) -> int:
    """Tokens per KV split.  One CTA covers one split of one sequence (all kv
    heads, so `num_kv_heads` does not enter): aim for a few waves of CTAs, keep a
    split at least 128 tokens so the pipeline fill is amortised, at most 1024 so
    ragged lengths still balance."""
    if batch <= 96:
        # few sequences: the per-CTA fixed cost dominates, so splits are as long as still fills the GPU -
        # about 1.75 CTAs per SM over the batch's expected tokens (1 024 at 64 rows of up to 8 192 tokens, the
        # measured optimum; 128 for 16 rows of 4 096, where 1 024 would leave half the SMs idle)
        tokens = batch * max(1, max_ctx // 2)
        split = (tokens * 4 + 7 * num_sms - 1) // (7 * num_sms)
        return int(min(1024, max(128, ((split + 63) // 64) * 64)))
    target_ctas = 6 * num_sms
    per_seq = max(1, target_ctas // max(1, batch))
    split = (max_ctx // 2 + per_seq - 1) // per_seq  # typical row is about half the table width
    split = ((split + 63) // 64) * 64
    return int(min(max(split, 128), 1024))


def paged_attn_workspace(batch, num_q_heads, head_dim, max_pages, page_size, split_tokens, device):
    n = _lib.load().b200_paged_attn_workspace_bytes(batch, num_q_heads, head_dim, max_pages, page_size, split_tokens)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def paged_attn_decode(
    q: torch.Tensor,
    k_pool: torch.Tensor,
    v_pool: torch.Tensor,
    block_table: torch.Tensor,
    ctx_lens: torch.Tensor,
    scale: float,
    split_tokens: int | None = None,
    workspace: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    pairs: bool = False,
) -> torch.Tensor:
    """softmax(q K^T * scale) V over the pages listed in `block_table`.

    q [B, Hq, D]; pools [num_blocks, Hkv, page, D] (the reference BlockManager
    layout); block_table [B, max_pages] int32; ctx_lens [B] int32.
    `pairs`: rows 2i and 2i+1 are consecutive tokens of one sequence and share table row 2i (a prompt chunk);
    every page is then fetched once for the two rows.  See `paged_attn_pairs_supported`.
    """
    _need(q, "q")
    _need(k_pool, "k_pool", q.dtype)
    _need(v_pool, "v_pool", q.dtype)
    _need(block_table, "block_table", torch.int32)
    _need(ctx_lens, "ctx_lens", torch.int32)
    if q.dtype not in DTYPE_CODE:
        raise ValueError(f"unsupported dtype {q.dtype}")
    B, Hq, D = q.shape
    nb, Hkv, page, D2 = k_pool.shape
    if D2 != D or v_pool.shape != k_pool.shape:
        raise ValueError("pool shape does not match q / each other")
    if block_table.shape[0] != B or ctx_lens.shape[0] != B:
        raise ValueError("block_table / ctx_lens batch mismatch")
    max_pages = block_table.shape[1]
    if split_tokens is None:
        split_tokens = default_split_tokens(B, Hkv, max_pages * page)
    if workspace is None:
        workspace = paged_attn_workspace(B, Hq, D, max_pages, page, split_tokens, q.device)
    if out is None:
        out = torch.empty_like(q)
    if pairs:
        rc = _lib.load().b200_paged_attn_decode_pairs(
            _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(ctx_lens), _ptr(out),
            _ptr(workspace), workspace.numel(), B, Hq, Hkv, D, page, nb, max_pages, float(scale),
            int(split_tokens), _stream(),
        )
        check(rc, "b200_paged_attn_decode_pairs")
        return out
    rc = _lib.load().b200_paged_attn_decode(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(ctx_lens), _ptr(out),
        _ptr(workspace), workspace.numel(), B, Hq, Hkv, D, page, nb, max_pages, float(scale),
        int(split_tokens), DTYPE_CODE[q.dtype], _stream(),
    )
    check(rc, "b200_paged_attn_decode")
    return out


def paged_attn_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, table_row: torch.Tensor,
                       first_pos: int, scale: float, status: torch.Tensor | None = None,
                       out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of a chunk of consecutive prompt tokens of one sequence over its pages.

    q [R, Hq, D] (positions first_pos .. first_pos + R - 1, K/V already in their page slots); table_row
    [max_pages] int32.  See `paged_attn_prefill_supported`."""
    _need(q, "q", torch.bfloat16)
    _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16)
    _need(table_row, "table_row", torch.int32)
    R, Hq, D = q.shape
    nb, Hkv, page, D2 = k_pool.shape
    if D2 != D or v_pool.shape != k_pool.shape:
        raise ValueError("pool shape does not match q / each other")
    if out is None:
        out = torch.empty_like(q)
    rc = _lib.load().b200_paged_attn_prefill(_ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(table_row), _ptr(out),
                                             _ptr(status), R, int(first_pos), Hq, Hkv, D, page, nb,
                                             table_row.numel(), float(scale), _stream())
    check(rc, "b200_paged_attn_prefill")
    return out


def paged_attn_prefill_supported(num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, dtype) -> bool:
    """Whether b200_paged_attn_prefill is built for this shape."""
    if dtype != torch.bfloat16 or page_size != 16 or num_q_heads % num_kv_heads:
        return False
    return (head_dim, num_q_heads // num_kv_heads) in ((128, 8), (128, 16), (64, 4))


def paged_attn_pairs_supported(num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, dtype) -> bool:
    """Whether b200_paged_attn_decode_pairs is built for this shape."""
    return (dtype == torch.bfloat16 and page_size == 16 and num_q_heads % num_kv_heads == 0
            and num_q_heads // num_kv_heads <= 8 and (head_dim, num_kv_heads) in ((128, 4), (64, 2)))


def kv_append(k_new, v_new, k_pool, v_pool, block_table, positions, status: torch.Tensor | None = None):
    """Write this step's K/V rows [B, Hkv, D] into page slot `positions[b]` of each row."""
    _need(k_new, "k_new", k_pool.dtype)
    _need(v_new, "v_new", k_pool.dtype)
    _need(k_pool, "k_pool")
    _need(v_pool, "v_pool", k_pool.dtype)
    _need(block_table, "block_table", torch.int32)
    _need(positions, "positions", torch.int32)
    B, Hkv, D = k_new.shape
    nb, Hkv2, page, D2 = k_pool.shape
    if (Hkv2, D2) != (Hkv, D):
        raise ValueError("k_new does not match the pool layout")
    rc = _lib.load().b200_kv_append(
        _ptr(k_new), _ptr(v_new), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), _ptr(positions),
        _ptr(status), B, Hkv, D, page, nb, block_table.shape[1], DTYPE_CODE[k_pool.dtype], _stream(),
    )
    check(rc, "b200_kv_append")


# ---------------------------------------------------------- dense projections


def dense_gemm_workspace(num_rows: int, out_features: int, device) -> torch.Tensor:
    """Room for the fp32 partial tiles of a K-split product of up to `num_rows` x `out_features`."""
    n = _lib.load().b200_dense_gemm_workspace_bytes(int(num_rows), int(out_features))
    return torch.empty(max(n, 16), dtype=torch.uint8, device=device)


def dense_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, status: torch.Tensor | None = None,
               k_split: int = 0, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """y = x w^T for bf16 x [M, K] and w [N, K] (fp32 accumulation, bf16 result).  Callers on a hot path pass a
    `workspace` (dense_gemm_workspace) that they keep; without one it is allocated here when a K split is used."""
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    M, K = x.shape
    N, K2 = w.shape
    if K2 != K:
        raise ValueError(f"x has {K} columns, w has {K2}")
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    _need(out, "out", torch.bfloat16)
    if M == 0:
        return out
    if workspace is None and k_split != 1:
        if k_split == 0 and ((N + 127) // 128) * ((M + 255) // 256) >= 128:
            k_split = 1  # enough weight tiles to fill the GPU: the library would not split either
        else:
            workspace = dense_gemm_workspace(M, N, x.device)
    rc = _lib.load().b200_dense_gemm_bf16(_ptr(x), _ptr(w), _ptr(out), _ptr(workspace),
                                          0 if workspace is None else workspace.numel(), _ptr(status), M, N, K,
                                          int(k_split), _stream())
    check(rc, "b200_dense_gemm_bf16")
    return out


def qkv_rope_append_supported(head_dim: int, in_features: int) -> bool:
    return bool(_lib.load().b200_qkv_rope_append_supported(int(head_dim), int(in_features)))


def qkv_rope_append_gemm(x, wqkv, q_norm_w, k_norm_w, cos, sin, positions, block_table, k_pool, v_pool, num_q_heads,
                         eps: float, status=None, q_out=None) -> torch.Tensor:
    """The q/k/v projection with per-head q/k RMSNorm, RoPE and the K/V page write in its epilogue: q returned
    [rows, Hq, 128], k and v written into their page slots.  dense_gemm + qk_norm_rope_append in one kernel."""
    _need(x, "x", torch.bfloat16)
    _need(wqkv, "wqkv", torch.bfloat16)
    _need(cos, "cos", torch.bfloat16)
    _need(sin, "sin", torch.bfloat16)
    _need(positions, "positions", torch.int32)
    _need(block_table, "block_table", torch.int32)
    _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16)
    R, K = x.shape
    nb, Hkv, page, D = k_pool.shape
    if wqkv.shape != ((num_q_heads + 2 * Hkv) * D, K):
        raise ValueError("wqkv does not match the heads and the input width")
    if q_out is None:
        q_out = torch.empty(R, num_q_heads, D, dtype=torch.bfloat16, device=x.device)
    if R == 0:
        return q_out
    rc = _lib.load().b200_qkv_rope_append_gemm(
        _ptr(x), _ptr(wqkv), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(block_table),
        _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(status), R, num_q_heads, Hkv, D, K, float(eps), page, nb,
        block_table.shape[1], cos.shape[0], _stream())
    check(rc, "b200_qkv_rope_append_gemm")
    return q_out


def lm_head_argmax_workspace(device) -> torch.Tensor:
    return torch.zeros(_lib.load().b200_lm_head_argmax_workspace_bytes(), dtype=torch.uint8, device=device)


def lm_head_argmax(x: torch.Tensor, w: torch.Tensor, workspace: torch.Tensor | None = None,
                   out: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """argmax_n (x w^T)[m, n] per row without writing the logits; ties go to the lower index.  int64 [M]."""
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    M, K = x.shape
    if w.shape[1] != K:
        raise ValueError(f"x has {K} columns, w has {w.shape[1]}")
    if workspace is None:
        workspace = lm_head_argmax_workspace(x.device)
    if out is None:
        out = torch.empty(M, dtype=torch.int64, device=x.device)
    _need(out, "out", torch.int64)
    for lo in range(0, M, 256):  # the kernel keeps one running candidate per row in registers: 256 rows a call
        hi = min(M, lo + 256)
        rc = _lib.load().b200_lm_head_argmax(_ptr(x[lo:hi]), _ptr(w), out[lo:hi].data_ptr(), _ptr(workspace),
                                             workspace.numel(), _ptr(status), hi - lo, w.shape[0], K, _stream())
        check(rc, "b200_lm_head_argmax")
    return out


# ------------------------------------------------------------ fused step glue


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """x += delta (in place, when given); returns weight * rmsnorm(x)."""
    _need(x, "x", torch.bfloat16)
    _need(weight, "weight", torch.bfloat16)
    if delta is not None:
        _need(delta, "delta", torch.bfloat16)
    rows, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    rc = _lib.load().b200_add_rmsnorm(_ptr(x), _ptr(delta), _ptr(weight), float(eps), rows, H, _ptr(out), _stream())
    check(rc, "b200_add_rmsnorm")
    return out


def add_rmsnorm_route_supported(hidden: int, num_experts: int, top_k: int) -> bool:
    return bool(_lib.load().b200_add_rmsnorm_route_supported(int(hidden), int(num_experts), int(top_k)))


def add_rmsnorm_route(x: torch.Tensor, delta: torch.Tensor | None, norm_weight: torch.Tensor, eps: float,
                      router_weight: torch.Tensor, top_k: int, renormalize: bool = True,
                      num_valid: torch.Tensor | None = None, want_logits: bool = False):
    """x += delta (in place); h = norm_weight * rmsnorm(x); fp32 router logits h W_r^T; top-k routing - one
    kernel.  Returns (h bf16 [T, H], ids int32 [T, K], weights fp32 [T, K]) and, with want_logits, the fp32
    logits [T, E] as a fourth value."""
    _need(x, "x", torch.bfloat16)
    _need(norm_weight, "norm_weight", torch.bfloat16)
    _need(router_weight, "router_weight", torch.bfloat16)
    if delta is not None:
        _need(delta, "delta", torch.bfloat16)
    if num_valid is not None:
        _need(num_valid, "num_valid", torch.int32)
    T, H = x.shape
    E = router_weight.shape[0]
    if router_weight.shape[1] != H:
        raise ValueError("router_weight does not match the hidden size")
    h = torch.empty_like(x)
    ids = torch.empty(T, top_k, dtype=torch.int32, device=x.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=x.device)
    logits = torch.empty(T, E, dtype=torch.float32, device=x.device) if want_logits else None
    rc = _lib.load().b200_add_rmsnorm_route(_ptr(x), _ptr(delta), _ptr(norm_weight), float(eps), _ptr(router_weight), T, H,
                                            E, top_k, int(renormalize), _ptr(num_valid), _ptr(h), _ptr(ids), _ptr(w),
                                            _ptr(logits), _stream())
    check(rc, "b200_add_rmsnorm_route")
    return (h, ids, w, logits) if want_logits else (h, ids, w)


def qk_norm_rope_append(qkv, q_norm_w, k_norm_w, cos, sin, positions, block_table, k_pool, v_pool, num_q_heads,
                        eps: float, status=None, q_out=None) -> torch.Tensor:
    """Per-head q/k RMSNorm + RoPE; q returned [B, Hq, D], k and v written into their page slots."""
    _need(qkv, "qkv", torch.bfloat16)
    _need(cos, "cos", torch.bfloat16)
    _need(sin, "sin", torch.bfloat16)
    _need(positions, "positions", torch.int32)
    _need(block_table, "block_table", torch.int32)
    _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16)
    B, heads, D = qkv.shape
    nb, Hkv, page, D2 = k_pool.shape
    if D2 != D or heads != num_q_heads + 2 * Hkv:
        raise ValueError("qkv does not match the pool layout")
    if q_out is None:
        q_out = torch.empty(B, num_q_heads, D, dtype=torch.bfloat16, device=qkv.device)
    rc = _lib.load().b200_qk_norm_rope_append(
        _ptr(qkv), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos), _ptr(sin), _ptr(positions), _ptr(block_table),
        _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(status), B, num_q_heads, Hkv, D, float(eps), page, nb,
        block_table.shape[1], cos.shape[0], _stream())
    check(rc, "b200_qk_norm_rope_append")
    return q_out


# ------------------------------------------------------------------------ MoE


def moe_route(logits: torch.Tensor, top_k: int, renormalize: bool = True, num_valid: torch.Tensor | None = None):
    """fp32 softmax top-k routing on fp32 or bf16 logits. Returns (ids [T,K] int32, weights [T,K] fp32).
    `num_valid` (device int32 scalar): rows at or beyond it get id -1 and weight 0 (padding rows)."""
    _need(logits, "logits")
    if num_valid is not None:
        _need(num_valid, "num_valid", torch.int32)
    if logits.dtype not in DTYPE_CODE:
        raise ValueError(f"logits must be float32 or bfloat16, got {logits.dtype}")
    T, E = logits.shape
    ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    rc = _lib.load().b200_moe_route(_ptr(logits), DTYPE_CODE[logits.dtype], T, E, top_k, int(renormalize),
                                    _ptr(num_valid), _ptr(ids), _ptr(w), _stream())
    check(rc, "b200_moe_route")
    return ids, w


class Permutation:
    """Result of moe_permute: the stable sort of (token, slot) pairs by expert."""

    __slots__ = ("sorted_pair_ids", "row_of_pair", "expert_offsets", "tiles", "num_tiles", "workspace")


def new_permutation(num_tokens: int, top_k: int, num_experts: int, device) -> Permutation:
    """Buffers of one permutation.  Callers on a hot path allocate them once and pass them as `perm=`; the
    workspace starts zeroed (its first word is the sticky device status)."""
    lib = _lib.load()
    n = num_tokens * top_k
    p = Permutation()
    p.sorted_pair_ids = torch.empty(n, dtype=torch.int32, device=device)
    p.row_of_pair = torch.empty(n, dtype=torch.int32, device=device)
    p.expert_offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=device)
    p.tiles = torch.zeros(max(1, lib.b200_moe_max_tiles(num_tokens, num_experts, top_k)), 4, dtype=torch.int32, device=device)
    p.num_tiles = torch.zeros(1, dtype=torch.int32, device=device)
    p.workspace = torch.zeros(lib.b200_moe_permute_workspace_bytes(num_tokens, num_experts, top_k), dtype=torch.uint8,
                              device=device)
    return p


def moe_permute(topk_ids: torch.Tensor, num_experts: int, tile_experts: int = 0, perm: Permutation | None = None) -> Permutation:
    """Stable sort of the (token, slot) pairs by expert id; only experts below `tile_experts` (0 = all) get
    row tiles for the grouped GEMM."""
    _need(topk_ids, "topk_ids", torch.int32)
    T, K = topk_ids.shape
    lib = _lib.load()
    p = perm if perm is not None else new_permutation(T, K, num_experts, topk_ids.device)
    rc = lib.b200_moe_permute(
        _ptr(topk_ids), T, num_experts, K, _ptr(p.sorted_pair_ids), _ptr(p.row_of_pair),
        _ptr(p.expert_offsets), _ptr(p.tiles), _ptr(p.num_tiles), int(tile_experts), _ptr(p.workspace),
        p.workspace.numel(), _stream(),
    )
    check(rc, "b200_moe_permute")
    return p


def moe_permute_quant(topk_ids: torch.Tensor, x: torch.Tensor, num_experts: int):
    """moe_permute + act_quant_fp8 in one pass. Returns (Permutation, xq, x_scale)."""
    _need(topk_ids, "topk_ids", torch.int32)
    _need(x, "x", torch.bfloat16)
    T, K = topk_ids.shape
    H = x.shape[1]
    lib = _lib.load()
    dev = x.device
    p = Permutation()
    p.sorted_pair_ids = torch.empty(T * K, dtype=torch.int32, device=dev)
    p.row_of_pair = torch.empty(T * K, dtype=torch.int32, device=dev)
    p.expert_offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    p.tiles = torch.zeros(max(1, lib.b200_moe_max_tiles(T, num_experts, K)), 4, dtype=torch.int32, device=dev)
    p.num_tiles = torch.zeros(1, dtype=torch.int32, device=dev)
    p.workspace = torch.zeros(lib.b200_moe_permute_workspace_bytes(T, num_experts, K), dtype=torch.uint8, device=dev)
    xq = torch.empty(T * K, H, dtype=torch.uint8, device=dev)
    xs = torch.empty(T * K, H // 128, dtype=torch.float32, device=dev)
    rc = lib.b200_moe_permute_quant(
        _ptr(topk_ids), _ptr(x), T, num_experts, K, H, _ptr(p.sorted_pair_ids), _ptr(p.row_of_pair),
        _ptr(p.expert_offsets), _ptr(p.tiles), _ptr(p.num_tiles), _ptr(xq), _ptr(xs), _ptr(p.workspace),
        p.workspace.numel(), _stream())
    check(rc, "b200_moe_permute_quant")
    return p, xq, xs


def moe_permute_quant_ep(topk_ids, x, num_experts: int, ep_world: int, ep_capacity: int, xq_send, xs_send,
                         expert_of_slot, overflow, perm: Permutation | None = None, slot_of_pair=None):
    """Expert-parallel dispatch side: sort, quantise and place every row in its send slot.
    `expert_of_slot` gets the owner-local expert id of every used slot and the empty id (num_experts //
    ep_world) of every other; `overflow` is an int32 flag.
    Returns (Permutation, slot_of_pair int32 [T*K])."""
    _need(topk_ids, "topk_ids", torch.int32)
    _need(x, "x", torch.bfloat16)
    _need(xq_send, "xq_send", torch.uint8)
    _need(xs_send, "xs_send", torch.float32)
    _need(expert_of_slot, "expert_of_slot", torch.int32)
    _need(overflow, "overflow", torch.int32)
    T, K = topk_ids.shape
    H = x.shape[1]
    if xq_send.shape[0] < ep_world * ep_capacity or expert_of_slot.numel() < ep_world * ep_capacity:
        raise ValueError("send buffers are smaller than ep_world * ep_capacity rows")
    lib = _lib.load()
    dev = x.device
    p = perm if perm is not None else new_permutation(T, K, num_experts, dev)
    if slot_of_pair is None:
        slot_of_pair = torch.empty(T * K, dtype=torch.int32, device=dev)
    rc = lib.b200_moe_permute_quant_ep(
        _ptr(topk_ids), _ptr(x), T, num_experts, K, H, ep_world, ep_capacity, _ptr(p.sorted_pair_ids),
        _ptr(p.row_of_pair), _ptr(p.expert_offsets), _ptr(p.tiles), _ptr(p.num_tiles), _ptr(xq_send), _ptr(xs_send),
        _ptr(slot_of_pair), _ptr(expert_of_slot), _ptr(overflow), _ptr(p.workspace), p.workspace.numel(), _stream())
    check(rc, "b200_moe_permute_quant_ep")
    return p, slot_of_pair


def _ptr_array(ptrs):
    """Host array of device pointers (ints) for the *_peers arguments."""
    import ctypes
    return (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def moe_permute_quant_ep_p2p(topk_ids, x, num_experts: int, ep_world: int, ep_capacity: int, ep_rank: int,
                             xq_peers, xs_peers, id_peers, overflow, perm: Permutation | None = None,
                             slot_of_pair=None):
    """moe_permute_quant_ep writing rows, scales and ids straight into the owners' receive buffers.
    `*_peers` are lists of ep_world device addresses (entry r = that buffer of rank r as mapped here).
    Returns (Permutation, slot_of_pair int32 [T*K])."""
    _need(topk_ids, "topk_ids", torch.int32)
    _need(x, "x", torch.bfloat16)
    _need(overflow, "overflow", torch.int32)
    if not (len(xq_peers) == len(xs_peers) == len(id_peers) == ep_world):
        raise ValueError("need one peer address per rank")
    T, K = topk_ids.shape
    H = x.shape[1]
    lib = _lib.load()
    dev = x.device
    p = perm if perm is not None else new_permutation(T, K, num_experts, dev)
    if slot_of_pair is None:
        slot_of_pair = torch.empty(T * K, dtype=torch.int32, device=dev)
    rc = lib.b200_moe_permute_quant_ep_p2p(
        _ptr(topk_ids), _ptr(x), T, num_experts, K, H, ep_world, ep_capacity, ep_rank, _ptr(p.sorted_pair_ids),
        _ptr(p.row_of_pair), _ptr(p.expert_offsets), _ptr(p.tiles), _ptr(p.num_tiles), _ptr_array(xq_peers),
        _ptr_array(xs_peers), _ptr_array(id_peers), _ptr(slot_of_pair), _ptr(overflow), _ptr(p.workspace),
        p.workspace.numel(), _stream())
    check(rc, "b200_moe_permute_quant_ep_p2p")
    return p, slot_of_pair


def ep_signal(flag_peers, epoch: torch.Tensor, ep_rank: int, ep_world: int):
    _need(epoch, "epoch", torch.int32)
    check(_lib.load().b200_ep_signal(_ptr_array(flag_peers), _ptr(epoch), ep_rank, ep_world, _stream()), "b200_ep_signal")


def ep_wait(local_flags: torch.Tensor, epoch: torch.Tensor, ep_world: int, status: torch.Tensor | None = None):
    _need(local_flags, "local_flags", torch.int32)
    _need(epoch, "epoch", torch.int32)
    check(_lib.load().b200_ep_wait(_ptr(local_flags), _ptr(epoch), ep_world, _ptr(status), _stream()), "b200_ep_wait")


def ep_barrier(flag_peers, epoch: torch.Tensor, ep_rank: int, ep_world: int, status: torch.Tensor | None = None):
    _need(epoch, "epoch", torch.int32)
    check(_lib.load().b200_ep_barrier(_ptr_array(flag_peers), _ptr(epoch), ep_rank, ep_world, _ptr(status), _stream()),
          "b200_ep_barrier")


def ipc_export(t: torch.Tensor):
    """(64-byte handle, offset) that another process of the node can map with ipc_import."""
    import ctypes
    _need(t, "tensor")
    handle = ctypes.create_string_buffer(64)
    off = ctypes.c_uint64(0)
    check(_lib.load().b200_ipc_export(_ptr(t), handle, ctypes.byref(off)), "b200_ipc_export")
    return bytes(handle.raw), int(off.value)


def ipc_import(handle: bytes, offset: int):
    """Maps an exported allocation; returns (base address for ipc_close, address of the exported tensor)."""
    import ctypes
    base, ptr = ctypes.c_void_p(0), ctypes.c_void_p(0)
    buf = ctypes.create_string_buffer(handle, 64)
    check(_lib.load().b200_ipc_import(buf, offset, ctypes.byref(base), ctypes.byref(ptr)), "b200_ipc_import")
    return int(base.value), int(ptr.value)


def ipc_close(base: int):
    check(_lib.load().b200_ipc_close(base), "b200_ipc_close")


def moe_permute_gather_fp8(ids, num_experts: int, tile_experts: int, src_q, src_scale, dst_q, dst_scale,
                           perm: Permutation | None = None) -> Permutation:
    """Receive side of the expert-parallel exchange: sort the received rows by their (local) expert id and
    copy them into that order, in one pass.  Experts >= tile_experts are ranked but neither tiled nor copied."""
    _need(ids, "ids", torch.int32)
    _need(src_q, "src_q", torch.uint8)
    _need(src_scale, "src_scale", torch.float32)
    _need(dst_q, "dst_q", torch.uint8)
    _need(dst_scale, "dst_scale", torch.float32)
    n, H = ids.numel(), src_q.shape[1]
    p = perm if perm is not None else new_permutation(n, 1, num_experts, ids.device)
    rc = _lib.load().b200_moe_permute_gather_fp8(
        _ptr(ids), n, num_experts, tile_experts, _ptr(src_q), _ptr(src_scale), H, _ptr(p.sorted_pair_ids),
        _ptr(p.row_of_pair), _ptr(p.expert_offsets), _ptr(p.tiles), _ptr(p.num_tiles), _ptr(dst_q), _ptr(dst_scale),
        _ptr(p.workspace), p.workspace.numel(), _stream())
    check(rc, "b200_moe_permute_gather_fp8")
    return p


def gather_rows_fp8(src_q, src_scale, order, dst_q=None, dst_scale=None):
    """dst row i = src row order[i] for e4m3 rows and their per-128 scales."""
    _need(src_q, "src_q", torch.uint8)
    _need(src_scale, "src_scale", torch.float32)
    _need(order, "order", torch.int32)
    n, H = order.numel(), src_q.shape[1]
    if dst_q is None:
        dst_q = torch.empty(n, H, dtype=torch.uint8, device=src_q.device)
    if dst_scale is None:
        dst_scale = torch.empty(n, H // 128, dtype=torch.float32, device=src_q.device)
    rc = _lib.load().b200_gather_rows_fp8(_ptr(src_q), _ptr(src_scale), _ptr(order), n, H, _ptr(dst_q), _ptr(dst_scale),
                                          _stream())
    check(rc, "b200_gather_rows_fp8")
    return dst_q, dst_scale


def act_quant_fp8(x: torch.Tensor, row_of_pair: torch.Tensor | None = None, top_k: int = 1):
    """Per-row, per-128-column e4m3 quantisation; optionally scattered to sorted rows.

    Returns (xq uint8 [rows, H], scale fp32 [rows, H/128])."""
    _need(x, "x", torch.bfloat16)
    T, H = x.shape
    rows = T if row_of_pair is None else T * top_k
    xq = torch.empty(rows, H, dtype=torch.uint8, device=x.device)
    xs = torch.empty(rows, H // 128, dtype=torch.float32, device=x.device)
    rc = _lib.load().b200_act_quant_fp8(_ptr(x), _ptr(row_of_pair), T, H, top_k, _ptr(xq), _ptr(xs), _stream())
    check(rc, "b200_act_quant_fp8")
    return xq, xs


def _as_u8(t: torch.Tensor) -> torch.Tensor:
    return t.view(torch.uint8) if t.dtype != torch.uint8 else t


def _weight_dims(w: torch.Tensor):
    """(num_experts, rows, cols, layout code) of an expert weight tensor: 3-D [E, rows, cols] is the
    row-major checkpoint layout, 5-D [E, rows/128, cols/128, 128, 128] the tiled one (quant.tile_weight_blocks)."""
    if w.dim() == 3:
        return w.shape[0], w.shape[1], w.shape[2], 0
    if w.dim() == 5 and w.shape[3] == 128 and w.shape[4] == 128:
        return w.shape[0], w.shape[1] * 128, w.shape[2] * 128, 1
    raise ValueError(f"expert weights must be [E, rows, cols] or [E, rows/128, cols/128, 128, 128], got {tuple(w.shape)}")


def moe_fp8_gemm_gate_up(xq, x_scale, w13, w13_scale_inv, perm: Permutation, status=None):
    """h = silu(W13[:I] x) * (W13[I:] x) per sorted row, re-quantised to e4m3."""
    xq, w13 = _as_u8(xq), _as_u8(w13)
    _need(xq, "xq", torch.uint8)
    _need(w13, "w13", torch.uint8)
    _need(x_scale, "x_scale", torch.float32)
    _need(w13_scale_inv, "w13_scale_inv", torch.float32)
    rows, H = xq.shape
    E, two_i, H2, layout = _weight_dims(w13)
    inter = two_i // 2
    if H2 != H or tuple(w13_scale_inv.shape) != (E, two_i // 128, H // 128):
        raise ValueError("w13 / scale shapes do not match")
    hq = torch.empty(rows, inter, dtype=torch.uint8, device=xq.device)
    hs = torch.empty(rows, inter // 128, dtype=torch.float32, device=xq.device)
    rc = _lib.load().b200_moe_fp8_gemm_gate_up(
        _ptr(xq), _ptr(x_scale), _ptr(w13), _ptr(w13_scale_inv), _ptr(perm.tiles), _ptr(perm.num_tiles),
        _ptr(hq), _ptr(hs), _ptr(status), rows, E, H, inter, layout, _stream(),
    )
    check(rc, "b200_moe_fp8_gemm_gate_up")
    return hq, hs


def moe_fp8_gemm_down(hq, h_scale, w2, w2_scale_inv, perm: Permutation, status=None, out=None, out_row_map=None):
    """y = W2 h per sorted row, bf16.  With `out_row_map` (int32 per sorted row) row r is written to row
    out_row_map[r] of `out` instead of row r."""
    hq, w2 = _as_u8(hq), _as_u8(w2)
    _need(hq, "hq", torch.uint8)
    _need(w2, "w2", torch.uint8)
    _need(h_scale, "h_scale", torch.float32)
    _need(w2_scale_inv, "w2_scale_inv", torch.float32)
    rows, inter = hq.shape
    E, H, inter2, layout = _weight_dims(w2)
    if inter2 != inter or tuple(w2_scale_inv.shape) != (E, H // 128, inter // 128):
        raise ValueError("w2 / scale shapes do not match")
    if out_row_map is not None:
        _need(out_row_map, "out_row_map", torch.int32)
    y = out if out is not None else torch.empty(rows, H, dtype=torch.bfloat16, device=hq.device)
    _need(y, "out", torch.bfloat16)
    rc = _lib.load().b200_moe_fp8_gemm_down(
        _ptr(hq), _ptr(h_scale), _ptr(w2), _ptr(w2_scale_inv), _ptr(perm.tiles), _ptr(perm.num_tiles),
        _ptr(y), _ptr(out_row_map), _ptr(status), rows, E, H, inter, layout, _stream(),
    )
    check(rc, "b200_moe_fp8_gemm_down")
    return y


def moe_fp8_gemm_down_p2p(hq, h_scale, w2, w2_scale_inv, perm: Permutation, y_peers, out_row_map, ep_world: int,
                          ep_capacity: int, ep_rank: int, status=None):
    """Down GEMM whose epilogue writes every row into y_recv of the rank the row came from (`y_peers`:
    ep_world device addresses); `out_row_map` gives the receive slot of each sorted row."""
    hq, w2 = _as_u8(hq), _as_u8(w2)
    _need(hq, "hq", torch.uint8)
    _need(w2, "w2", torch.uint8)
    _need(h_scale, "h_scale", torch.float32)
    _need(w2_scale_inv, "w2_scale_inv", torch.float32)
    _need(out_row_map, "out_row_map", torch.int32)
    rows, inter = hq.shape
    E, H, inter2, layout = _weight_dims(w2)
    if inter2 != inter or tuple(w2_scale_inv.shape) != (E, H // 128, inter // 128):
        raise ValueError("w2 / scale shapes do not match")
    if len(y_peers) != ep_world:
        raise ValueError("need one peer address per rank")
    rc = _lib.load().b200_moe_fp8_gemm_down_p2p(
        _ptr(hq), _ptr(h_scale), _ptr(w2), _ptr(w2_scale_inv), _ptr(perm.tiles), _ptr(perm.num_tiles),
        _ptr_array(y_peers), _ptr(out_row_map), _ptr(status), rows, E, H, inter, layout, ep_world, ep_capacity,
        ep_rank, _stream())
    check(rc, "b200_moe_fp8_gemm_down_p2p")


def moe_combine(y_sorted, row_of_pair, topk_weights):
    _need(y_sorted, "y_sorted", torch.bfloat16)
    _need(row_of_pair, "row_of_pair", torch.int32)
    _need(topk_weights, "topk_weights", torch.float32)
    T, K = topk_weights.shape
    H = y_sorted.shape[1]
    out = torch.empty(T, H, dtype=torch.bfloat16, device=y_sorted.device)
    rc = _lib.load().b200_moe_combine(_ptr(y_sorted), _ptr(row_of_pair), _ptr(topk_weights), T, H, K, _ptr(out), _stream())
    check(rc, "b200_moe_combine")
    return out


def moe_combine_add_rmsnorm(y_sorted, row_of_pair, topk_weights, x, weight, eps: float, out=None):
    """x += bf16(sum_k w * y) in place; returns weight * rmsnorm(x)."""
    _need(y_sorted, "y_sorted", torch.bfloat16)
    _need(row_of_pair, "row_of_pair", torch.int32)
    _need(topk_weights, "topk_weights", torch.float32)
    _need(x, "x", torch.bfloat16)
    _need(weight, "weight", torch.bfloat16)
    T, K = topk_weights.shape
    H = y_sorted.shape[1]
    if out is None:
        out = torch.empty_like(x)
    rc = _lib.load().b200_moe_combine_add_rmsnorm(_ptr(y_sorted), _ptr(row_of_pair), _ptr(topk_weights), _ptr(x),
                                                  _ptr(weight), float(eps), T, H, K, _ptr(out), _stream())
    check(rc, "b200_moe_combine_add_rmsnorm")
    return out


def moe_fp8_workspace(num_tokens, num_experts, top_k, hidden, inter, device):
    n = _lib.load().b200_moe_fp8_workspace_bytes(num_tokens, num_experts, top_k, hidden, inter)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def moe_fp8_forward(x, router_logits, w13, w13_scale_inv, w2, w2_scale_inv, top_k, renormalize=True,
                    workspace=None, out=None, residual=None, norm_weight=None, eps: float = 1e-6, routing=None):
    """The whole FP8 MoE layer on one stream: route, permute+quantise, two grouped GEMMs, combine.

    With `residual` and `norm_weight` the combine is fused with the next residual add and RMSNorm:
    `residual` is updated in place and the returned tensor is norm_weight * rmsnorm(residual).
    `routing` = (ids int32 [T, K], weights fp32 [T, K]) skips the router (tokens routed by
    add_rmsnorm_route); `router_logits` is then unused and the residual form is required."""
    w13, w2 = _as_u8(w13), _as_u8(w2)
    _need(x, "x", torch.bfloat16)
    if routing is not None:
        ids, wts = routing
        _need(ids, "routing ids", torch.int32)
        _need(wts, "routing weights", torch.float32)
        _need(w13, "w13", torch.uint8)
        _need(w2, "w2", torch.uint8)
        _need(residual, "residual", torch.bfloat16)
        _need(norm_weight, "norm_weight", torch.bfloat16)
        T, H = x.shape
        E, two_i, _, layout = _weight_dims(w13)
        if workspace is None:
            workspace = moe_fp8_workspace(T, E, top_k, H, two_i // 2, x.device)
        if out is None:
            out = torch.empty_like(x)
        rc = _lib.load().b200_moe_fp8_routed_add_rmsnorm(
            _ptr(x), _ptr(ids), _ptr(wts), _ptr(w13), _ptr(w13_scale_inv), _ptr(w2), _ptr(w2_scale_inv), _ptr(residual),
            _ptr(norm_weight), float(eps), _ptr(out), _ptr(workspace), workspace.numel(), T, E, top_k, H, two_i // 2,
            layout, _stream())
        check(rc, "b200_moe_fp8_routed_add_rmsnorm")
        return out
    _need(router_logits, "router_logits")
    if router_logits.dtype not in DTYPE_CODE:
        raise ValueError(f"router_logits must be float32 or bfloat16, got {router_logits.dtype}")
    _need(w13, "w13", torch.uint8)
    _need(w2, "w2", torch.uint8)
    _need(w13_scale_inv, "w13_scale_inv", torch.float32)
    _need(w2_scale_inv, "w2_scale_inv", torch.float32)
    T, H = x.shape
    E, two_i, _, layout = _weight_dims(w13)
    if _weight_dims(w2)[3] != layout:
        raise ValueError("w13 and w2 must use the same weight layout")
    inter = two_i // 2
    if workspace is None:
        workspace = moe_fp8_workspace(T, E, top_k, H, inter, x.device)
    if out is None:
        out = torch.empty_like(x)
    lib = _lib.load()
    ld = DTYPE_CODE[router_logits.dtype]
    if residual is None:
        rc = lib.b200_moe_fp8_forward(
            _ptr(x), _ptr(router_logits), ld, _ptr(w13), _ptr(w13_scale_inv), _ptr(w2), _ptr(w2_scale_inv),
            _ptr(out), _ptr(workspace), workspace.numel(), T, E, top_k, H, inter, int(renormalize), layout, _stream())
        check(rc, "b200_moe_fp8_forward")
    else:
        _need(residual, "residual", torch.bfloat16)
        _need(norm_weight, "norm_weight", torch.bfloat16)
        rc = lib.b200_moe_fp8_forward_add_rmsnorm(
            _ptr(x), _ptr(router_logits), ld, _ptr(w13), _ptr(w13_scale_inv), _ptr(w2), _ptr(w2_scale_inv),
            _ptr(residual), _ptr(norm_weight), float(eps), _ptr(out), _ptr(workspace), workspace.numel(), T, E,
            top_k, H, inter, int(renormalize), layout, _stream())
        check(rc, "b200_moe_fp8_forward_add_rmsnorm")
    return out
