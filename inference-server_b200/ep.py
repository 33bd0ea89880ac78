"""Expert-parallel dispatch planning (host/torch index arithmetic, no kernels).

Experts are partitioned by id: rank r of W owns experts [r*E/W, (r+1)*E/W).  Each
rank routes its own tokens, sorts the (token, slot) pairs by expert id (which is
also by destination rank) and exchanges rows with fixed-capacity all-to-alls so
that no step needs a host round trip:

    send buffer  [W, capacity, hidden]   slot s of segment d = the s-th pair of
                                         this rank that goes to rank d
    slot_of_pair [T*K]                   d * capacity + s for every pair
    expert_of_slot [W*capacity]          local expert id at the destination, or
                                         E_local for an empty slot

On the GPU the slot placement is done inside the scatter+quantise kernel
(``b200_moe_permute_quant_ep``); ``plan_dispatch`` is the same arithmetic in torch
ops, used by the CPU stand-in kernels of the gloo tests and as a cross-check.
"""
from __future__ import annotations

import torch


def default_capacity(num_tokens: int, top_k: int, world: int, factor: float = 2.0) -> int:
    """Rows reserved per (source, destination) pair: `factor` x the mean, rounded up to 16."""
    mean = num_tokens * top_k / world
    cap = int(mean * factor + 15) // 16 * 16
    return max(16, min(cap, num_tokens * top_k))


def plan_dispatch(topk_ids: torch.Tensor, row_of_pair: torch.Tensor, expert_offsets: torch.Tensor,
                  num_experts: int, world: int, capacity: int):
    """Index arrays for the fixed-capacity exchange.

    topk_ids [T, K] int32 (global expert ids), row_of_pair [T*K] int32 (position in the
    expert-sorted order), expert_offsets [E+1] int32.
    Returns (slot_of_pair [T*K] int64, expert_of_slot [W*capacity] int32, overflow scalar bool tensor).
    Pairs beyond `capacity` for a destination are dropped into slot -1 and flagged."""
    e_local = num_experts // world
    flat = topk_ids.reshape(-1).long()
    dst = flat // e_local
    seg_start = expert_offsets.long()[dst * e_local]
    pos = row_of_pair.long() - seg_start
    fits = pos < capacity
    overflow = (~fits).any()
    slot = torch.where(fits, dst * capacity + pos, torch.full_like(pos, -1))
    # fixed shapes only (the step is captured in a CUDA graph): overflowed pairs write to a spare last entry
    trash = world * capacity
    expert_of_slot = torch.full((trash + 1,), e_local, dtype=torch.int32, device=topk_ids.device)
    expert_of_slot.index_copy_(0, torch.where(fits, slot, torch.full_like(slot, trash)), (flat % e_local).to(torch.int32))
    expert_of_slot[trash:].fill_(e_local)  # (a fill kernel: a scalar assignment would be a host copy)
    return slot, expert_of_slot[:trash], overflow


class EPState:
    """Per-rank buffers of the expert-parallel exchange, allocated once (graph-capturable)."""

    def __init__(self, num_tokens: int, hidden: int, top_k: int, num_experts: int, world: int, capacity: int,
                 device, group=None):
        self.T, self.H, self.K, self.E, self.W, self.C = num_tokens, hidden, top_k, num_experts, world, capacity
        self.e_local = num_experts // world
        self.group = group
        rows = world * capacity
        u8, f32, i32 = torch.uint8, torch.float32, torch.int32
        self.xq_send = torch.zeros(rows, hidden, dtype=u8, device=device)
        self.xq_recv = torch.zeros(rows, hidden, dtype=u8, device=device)
        self.xs_send = torch.zeros(rows, hidden // 128, dtype=f32, device=device)
        self.xs_recv = torch.zeros(rows, hidden // 128, dtype=f32, device=device)
        self.id_send = torch.zeros(rows, dtype=i32, device=device)
        self.id_recv = torch.zeros(rows, dtype=i32, device=device)
        self.xq_sorted = torch.zeros(rows, hidden, dtype=u8, device=device)
        self.xs_sorted = torch.zeros(rows, hidden // 128, dtype=f32, device=device)
        self.y_send = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=device)
        self.y_recv = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=device)
        self.overflow = torch.zeros(1, dtype=i32, device=device)  # sticky: set when a destination's capacity ran out


def ep_moe_forward(st: EPState, h, logits, w13, w13_scale, w2, w2_scale, renormalize, kernels, all_to_all,
                   residual=None, norm_weight=None, eps: float = 1e-6):
    """One expert-parallel FP8 MoE layer on this rank's tokens `h` [T, H].

    `w13/w2` hold only this rank's experts.  `kernels` supplies the compute steps (the ``ops`` module on a
    GPU; a CPU stand-in in the gloo tests) and `all_to_all(out, inp)` the equal-split exchange.  Steps:
      1. route; sort by (global) expert id, quantise and place every row in its fixed-capacity send slot
         (one kernel: the sort by expert is also a sort by owner rank);
      2. all-to-all of e4m3 rows, scales and owner-local expert ids (empty slots carry the id E_local);
      3. stable sort of the received slots by local expert (the dummy expert E_local sorts last and gets no
         tiles), one gather into sorted order, grouped gate/up GEMM, down GEMM writing straight back into slot
         order;
      4. all-to-all back and weighted combine in the original (token, slot) order.
    Everything has fixed shapes and no host round trip, so the layer can sit inside a captured CUDA graph."""
    T, K, W, C, El = st.T, st.K, st.W, st.C, st.e_local
    ids, wts = kernels.moe_route(logits, K, renormalize)
    st.id_send.fill_(El)
    _, slot_of_pair = kernels.moe_permute_quant_ep(ids, h, st.E, W, C, st.xq_send, st.xs_send, st.id_send, st.overflow)
    all_to_all(st.xq_recv, st.xq_send)
    all_to_all(st.xs_recv, st.xs_send)
    all_to_all(st.id_recv, st.id_send)

    lperm = kernels.moe_permute(st.id_recv.view(-1, 1), El + 1, El)
    kernels.gather_rows_fp8(st.xq_recv, st.xs_recv, lperm.sorted_pair_ids, st.xq_sorted, st.xs_sorted)
    hq, hs = kernels.moe_fp8_gemm_gate_up(st.xq_sorted, st.xs_sorted, w13, w13_scale, lperm)
    kernels.moe_fp8_gemm_down(hq, hs, w2, w2_scale, lperm, out=st.y_send, out_row_map=lperm.sorted_pair_ids)
    all_to_all(st.y_recv, st.y_send)

    # pairs that overflowed (slot -1, flagged) contribute nothing
    rows = torch.clamp(slot_of_pair, min=0)
    wts = torch.where((slot_of_pair >= 0).view(T, K), wts, torch.zeros_like(wts))
    if residual is not None:
        return kernels.moe_combine_add_rmsnorm(st.y_recv, rows, wts, residual, norm_weight, eps)
    return kernels.moe_combine(st.y_recv, rows, wts)
