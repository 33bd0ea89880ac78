"""Oracle: MoE routing, permutation, FP8 block-scale arithmetic (test infrastructure only)."""
from __future__ import annotations

import numpy as np
import torch

FP8_MAX = 448.0


def route_ref(logits: torch.Tensor, top_k: int, renormalize: bool = True):
    """Router of transformers ``Qwen3MoeTopKRouter.forward`` (softmax in fp32 over
    experts, top-k, divide by the sum of the selected probabilities), with the
    tie rule fixed: value descending, equal values by lower expert id.  The order
    is taken on the logits (softmax is monotone); ``torch.topk`` on the
    probabilities gives the same ids wherever no two of the leading
    probabilities are equal.  Returns (ids int32 [T,K], weights fp32 [T,K])."""
    logits = logits.detach().cpu().float()
    order = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :top_k]
    probs = torch.softmax(logits, dim=-1, dtype=torch.float32)
    w = torch.gather(probs, 1, order)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return order.to(torch.int32), w


def permute_ref(topk_ids: torch.Tensor, num_experts: int):
    """Stable sort of the token-major (token, slot) pairs by expert id - the
    ``argsort`` + ``histc`` + ``cumsum`` step of transformers
    ``grouped_mm_experts_forward`` with the order made deterministic.
    Returns dict(sorted_pair_ids, row_of_pair, expert_offsets, tiles) as int32 numpy."""
    ids = topk_ids.detach().cpu().numpy().astype(np.int64).reshape(-1)
    sorted_pair = np.argsort(ids, kind="stable").astype(np.int32)
    row_of_pair = np.empty_like(sorted_pair)
    row_of_pair[sorted_pair] = np.arange(ids.size, dtype=np.int32)
    counts = np.bincount(ids, minlength=num_experts)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    tiles = []
    for e in range(num_experts):
        for j in range(0, int(counts[e]), 128):
            tiles.append((e, int(offsets[e]) + j, min(128, int(counts[e]) - j), 0))
    return dict(sorted_pair_ids=sorted_pair, row_of_pair=row_of_pair, expert_offsets=offsets,
                tiles=np.array(tiles, dtype=np.int32).reshape(-1, 4))


def quantize_weight_ref(w: torch.Tensor):
    """e4m3 weights + fp32 scale_inv per 128x128 tile, as transformers
    ``Fp8Quantize.convert``: scale = 448 / amax (1 if amax == 0),
    q = clamp(w * scale, +-448) -> e4m3, scale_inv = 1 / scale."""
    rows, cols = w.shape[-2:]
    lead = w.shape[:-2]
    t = w.detach().cpu().float().reshape(*lead, rows // 128, 128, cols // 128, 128)
    amax = t.abs().amax(dim=(-3, -1))
    safe = torch.where(amax > 0, amax, torch.ones_like(amax))
    scale = torch.where(amax > 0, FP8_MAX / safe, torch.ones_like(amax))
    q = (t * scale.unsqueeze(-1).unsqueeze(-3)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(w.shape), (1.0 / scale).float()


def dequant_weight(q: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    """w = q * scale_inv per 128x128 tile, scale_inv [..., rows/128, cols/128], as transformers
    ``Fp8Dequantize.convert`` (integrations/finegrained_fp8.py) - pinned bit-exact on its output by
    tests/golden/fp8_weight_dequant.npz."""
    rows, cols = q.shape[-2:]
    lead = q.shape[:-2]
    t = q.detach().cpu().float().reshape(*lead, rows // 128, 128, cols // 128, 128)
    return (t * scale_inv.detach().cpu().unsqueeze(-1).unsqueeze(-3)).reshape(q.shape)


def act_quant_ref(x: torch.Tensor):
    """Dynamic activation quantisation, one scale per row per 128 columns:
    s = amax / 448 (1 for an all-zero group), q = e4m3(x / s).  This is the
    published per-token-group rule of the FP8 block-scale inference kernels
    (``act_quant``: s = max|x| / 448, y = x / s).  Returns (e4m3 [R,C], fp32 [R,C/128])."""
    x = x.detach().cpu().float()
    R, C = x.shape
    g = x.reshape(R, C // 128, 128)
    amax = g.abs().amax(dim=-1)
    s = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (g / s.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(R, C), s


def dequant_act(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    R, C = q.shape
    return (q.detach().cpu().float().reshape(R, C // 128, 128) * s.detach().cpu().unsqueeze(-1)).reshape(R, C)


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).float()


def moe_fp8_ref(x, router_logits, w13_q, w13_s, w2_q, w2_s, top_k: int, renormalize: bool = True,
                return_parts: bool = False, hf_rounding: bool = False):
    """The FP8 expert layer on CPU.

    Follows transformers ``FP8Experts.forward`` / ``fp8_grouped_mm_experts_forward``:
    per (token, expert) pair  gate_up = W13 q(x)  (block-scaled product),
    h = silu(gate) * up (``_apply_gate``: first half of the rows is the gate),
    h re-quantised per row per 128, y = W2 q(h) (bf16), then
    out[t] = sum_k w[t,k] * y in fp32, rounded to bf16.  The block-scaled product
    equals dequant(A) @ dequant(W)^T up to fp32 rounding, which is how it is
    evaluated here.  One stated difference from that code: gate_up and h stay in
    fp32 until h is quantised (there they pass through bf16), which is the more
    accurate of the two and what the CUDA kernel does.  ``hf_rounding=True``
    evaluates the other form, with every rounding point of ``FP8Experts.forward``
    for a bf16 model: gate_up rounded to bf16 (``output_dtype=input.dtype``),
    ``act_fn(gate) * up`` as two bf16 operations, the routing weight cast to bf16
    and multiplied in bf16; tests bound the distance between the two forms.
    """
    ids, w = route_ref(router_logits, top_k, renormalize)
    return moe_fp8_experts_ref(x, ids, w, w13_q, w13_s, w2_q, w2_s, return_parts, hf_rounding)


def moe_fp8_experts_ref(x, ids, w, w13_q, w13_s, w2_q, w2_s, return_parts: bool = False, hf_rounding: bool = False):
    """The expert part of :func:`moe_fp8_ref` for given routing (ids int [T,K], weights fp32 [T,K]);
    this is the signature the model's experts module is called with
    (``experts(hidden_states, top_k_index, top_k_weights)``)."""
    x = x.detach().cpu()
    T, H = x.shape
    E = w13_q.shape[0]
    inter = w13_q.shape[1] // 2
    top_k = ids.shape[1]
    ids = ids.to(torch.int32)
    w = w.float()
    perm = permute_ref(ids, E)
    xq, xs = act_quant_ref(x)
    xd = dequant_act(xq, xs)
    sorted_pair = torch.from_numpy(perm["sorted_pair_ids"]).long()
    tok_of_row = sorted_pair // top_k
    off = perm["expert_offsets"]
    rows = T * top_k
    h_all = torch.zeros(rows, inter)
    y_all = torch.zeros(rows, H)
    hq_all = torch.zeros(rows, inter, dtype=torch.float8_e4m3fn)
    hs_all = torch.zeros(rows, inter // 128)
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi == lo:
            continue
        a = xd[tok_of_row[lo:hi]]
        w13 = dequant_weight(w13_q[e], w13_s[e])
        gu = a @ w13.t()
        if hf_rounding:
            gu = _bf16(gu)
        g, u = gu[:, :inter], gu[:, inter:]
        h = _bf16(_bf16(torch.nn.functional.silu(g)) * u) if hf_rounding else torch.nn.functional.silu(g) * u
        hq, hs = act_quant_ref(h)
        hq_all[lo:hi], hs_all[lo:hi] = hq, hs
        h_all[lo:hi] = h
        w2 = dequant_weight(w2_q[e], w2_s[e])
        y_all[lo:hi] = _bf16(dequant_act(hq, hs) @ w2.t())
    rop = torch.from_numpy(perm["row_of_pair"]).long().reshape(T, top_k)
    out = torch.zeros(T, H)
    for k in range(top_k):
        if hf_rounding:
            out = out + _bf16(y_all[rop[:, k]] * _bf16(w[:, k : k + 1]))
        else:
            out = out + w[:, k : k + 1] * y_all[rop[:, k]]
    out = out.to(torch.bfloat16)
    if return_parts:
        return out, dict(ids=ids, weights=w, perm=perm, xq=xq, xs=xs, h=h_all, hq=hq_all, hs=hs_all, y=y_all)
    return out


def moe_dense_ref(x, router_logits, gate_up_proj, down_proj, top_k: int, renormalize: bool = True):
    """Unquantised expert layer in fp32, following transformers
    ``Qwen3MoeExperts.forward`` (eager): per hit expert
    ``gate, up = linear(x, gate_up_proj[e]).chunk(2)``; ``silu(gate) * up``;
    ``linear(., down_proj[e])``; scaled by the routing weight and summed per
    token.  Used to pin the gate/up split, activation and combine against the
    installed module."""
    x = x.detach().cpu().float()
    T, H = x.shape
    E = gate_up_proj.shape[0]
    ids, w = route_ref(router_logits, top_k, renormalize)
    out = torch.zeros(T, H)
    for t in range(T):
        for k in range(top_k):
            e = int(ids[t, k])
            g, u = (gate_up_proj[e].float() @ x[t]).chunk(2)
            out[t] += w[t, k] * (down_proj[e].float() @ (torch.nn.functional.silu(g) * u))
    return out
