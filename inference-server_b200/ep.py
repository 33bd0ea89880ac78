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
    overflow = (pos >= capacity).any()
    slot = dst * capacity + pos
    slot = torch.where(pos < capacity, slot, torch.full_like(slot, -1))
    expert_of_slot = torch.full((world * capacity,), e_local, dtype=torch.int32, device=topk_ids.device)
    ok = slot >= 0
    expert_of_slot[slot[ok]] = (flat[ok] % e_local).to(torch.int32)
    return slot, expert_of_slot, overflow
