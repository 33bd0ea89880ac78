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

``plan_dispatch`` computes those index arrays with torch ops on whatever device
the inputs live on; it is shared by the GPU path and by the CPU (gloo) tests.
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
        # one spare row at the end of the send buffers takes the rows of pairs that overflow the capacity
        self._xq_send = torch.zeros(rows + 1, hidden, dtype=u8, device=device)
        self._xs_send = torch.zeros(rows + 1, hidden // 128, dtype=f32, device=device)
        self.xq_send, self.xs_send = self._xq_send[:rows], self._xs_send[:rows]
        self.xq_recv = torch.zeros(rows, hidden, dtype=u8, device=device)
        self.xs_recv = torch.zeros(rows, hidden // 128, dtype=f32, device=device)
        self.id_recv = torch.zeros(rows, dtype=i32, device=device)
        self.y_send = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=device)
        self.y_recv = torch.zeros(rows, hidden, dtype=torch.bfloat16, device=device)
        self.overflow = torch.zeros((), dtype=torch.bool, device=device)


def ep_moe_forward(st: EPState, h, logits, w13, w13_scale, w2, w2_scale, renormalize, kernels, all_to_all,
                   residual=None, norm_weight=None, eps: float = 1e-6):
    """One expert-parallel FP8 MoE layer on this rank's tokens `h` [T, H].

    `w13/w2` hold only this rank's experts.  `kernels` supplies the compute steps (the ``ops`` module on a
    GPU; a CPU stand-in in the gloo tests) and `all_to_all(out, inp)` the equal-split exchange.  Steps:
    route -> sort by (global) expert + quantise -> place rows in fixed-capacity send slots -> all-to-all of
    e4m3 rows, scales and local expert ids -> re-sort the received rows by local expert -> grouped GEMMs ->
    un-sort -> all-to-all back -> weighted combine in the original (token, slot) order."""
    T, K, W, C, El = st.T, st.K, st.W, st.C, st.e_local
    ids, wts = kernels.moe_route(logits, K, renormalize)
    perm, xq, xs = kernels.moe_permute_quant(ids, h, st.E)
    slot_of_pair, expert_of_slot, overflow = plan_dispatch(ids, perm.row_of_pair, perm.expert_offsets, st.E, W, C)
    st.overflow |= overflow
    slot_of_row = slot_of_pair[perm.sorted_pair_ids.long()]
    # rows that overflowed (flagged above) land in the spare row; the rest go to their slots
    dest = torch.where(slot_of_row >= 0, slot_of_row, torch.full_like(slot_of_row, W * C))
    st._xq_send.index_copy_(0, dest, xq)
    st._xs_send.index_copy_(0, dest, xs)
    all_to_all(st.xq_recv, st.xq_send)
    all_to_all(st.xs_recv, st.xs_send)
    all_to_all(st.id_recv, expert_of_slot.contiguous())

    # local experts: stable sort of the received slots by local expert id; empty slots carry id El and sort last
    lperm = kernels.moe_permute(st.id_recv.view(-1, 1), El + 1)
    n_real = ((lperm.tiles[:, 0] < El) & (torch.arange(lperm.tiles.shape[0], device=h.device) < lperm.num_tiles)).sum()
    lperm.num_tiles.copy_(n_real.to(torch.int32).view(1))
    order = lperm.sorted_pair_ids.long()
    xq_l = st.xq_recv.index_select(0, order)
    xs_l = st.xs_recv.index_select(0, order)
    hq, hs = kernels.moe_fp8_gemm_gate_up(xq_l, xs_l, w13, w13_scale, lperm)
    y_l = kernels.moe_fp8_gemm_down(hq, hs, w2, w2_scale, lperm)
    torch.index_select(y_l, 0, lperm.row_of_pair.long(), out=st.y_send)
    all_to_all(st.y_recv, st.y_send)

    rows = torch.where(slot_of_pair >= 0, slot_of_pair, torch.zeros_like(slot_of_pair)).to(torch.int32)
    wts = torch.where((slot_of_pair >= 0).view(T, K), wts, torch.zeros_like(wts))
    if residual is not None:
        return kernels.moe_combine_add_rmsnorm(st.y_recv, rows, wts, residual, norm_weight, eps)
    return kernels.moe_combine(st.y_recv, rows, wts)
