"""CPU stand-ins for the ``ops`` kernels, built from the oracle (test infrastructure only).

Same call signatures as ``inference-server_b200/ops.py`` for the functions the expert-parallel layer
uses, on CPU tensors, so the multi-rank host logic (slot planning, exchanges, re-sort, combine) can be
exercised with gloo ranks on a machine without a GPU."""
from __future__ import annotations

import types

import torch

from . import moe_ref


def moe_route(logits, top_k, renormalize=True, num_valid=None):
    ids, w = moe_ref.route_ref(logits.float(), top_k, renormalize)
    if num_valid is not None:  # padding rows of a fixed-shape pass: no expert, no weight
        n = int(num_valid)
        ids[n:] = -1
        w[n:] = 0
    return ids, w


def _perm(ids, num_experts):
    """Pairs with id -1 ("no expert") are left out: they sort behind every real pair and get row -1."""
    flat = ids.reshape(-1)
    real = flat >= 0
    n_real = int(real.sum())
    r = moe_ref.permute_ref(torch.where(real, flat, torch.full_like(flat, num_experts)).view(ids.shape), num_experts + 1)
    p = types.SimpleNamespace()
    p.sorted_pair_ids = torch.from_numpy(r["sorted_pair_ids"])
    p.row_of_pair = torch.from_numpy(r["row_of_pair"]).clone()
    p.row_of_pair[~real] = -1
    r["expert_offsets"] = r["expert_offsets"][: num_experts + 1]
    r["tiles"] = r["tiles"][r["tiles"][:, 0] < num_experts] if len(r["tiles"]) else r["tiles"]
    p.n_real = n_real
    p.expert_offsets = torch.from_numpy(r["expert_offsets"])
    tiles = torch.zeros(max(1, ids.numel() // 128 + num_experts), 4, dtype=torch.int32)
    tiles[: len(r["tiles"])] = torch.from_numpy(r["tiles"])
    p.tiles = tiles
    p.num_tiles = torch.tensor([len(r["tiles"])], dtype=torch.int32)
    return p


def moe_permute(ids, num_experts, tile_experts=0, perm=None):
    p = _perm(ids, num_experts)
    if tile_experts:
        n = int((p.tiles[: int(p.num_tiles), 0] < tile_experts).sum())
        p.num_tiles = torch.tensor([n], dtype=torch.int32)
    return p


def moe_permute_quant_ep(ids, x, num_experts, ep_world, ep_capacity, xq_send, xs_send, expert_of_slot, overflow,
                         perm=None, slot_of_pair=None):
    """Slot placement by the torch restatement in the package (ep.plan_dispatch), rows by the oracle quantiser."""
    import importlib

    ep = importlib.import_module("inference-server_b200.ep")
    p, xq, xs = moe_permute_quant(ids, x, num_experts)
    slot, eos, ovf = ep.plan_dispatch(ids, p.row_of_pair, p.expert_offsets, num_experts, ep_world, ep_capacity)
    slot_of_row = slot[p.sorted_pair_ids.long()]
    ok = slot_of_row >= 0
    xq_send[slot_of_row[ok]] = xq[ok]
    xs_send[slot_of_row[ok]] = xs[ok]
    expert_of_slot.copy_(eos)
    if bool(ovf):
        overflow.fill_(1)
    return p, slot.to(torch.int32)


def moe_permute_gather_fp8(ids, num_experts, tile_experts, src_q, src_s, dst_q, dst_s, perm=None):
    """Sort the received rows by local expert and copy them into that order (rows of experts >= tile_experts,
    the dummy expert of empty slots, are ranked but not copied)."""
    p = moe_permute(ids.view(-1, 1), num_experts, tile_experts)
    order = p.sorted_pair_ids.long()
    real = ids.view(-1)[order] < tile_experts
    dst_q[real] = src_q[order[real]]
    dst_s[real] = src_s[order[real]]
    return p


def gather_rows_fp8(src_q, src_s, order, dst_q, dst_s):
    dst_q.copy_(src_q[order.long()])
    dst_s.copy_(src_s[order.long()])
    return dst_q, dst_s


def moe_permute_quant(ids, x, num_experts):
    p = _perm(ids, num_experts)
    q, s = moe_ref.act_quant_ref(x)
    tok = p.sorted_pair_ids.long() // ids.shape[1]
    return p, q.view(torch.uint8)[tok].contiguous(), s[tok].contiguous()


def _rows_of_tiles(perm):
    n = int(perm.num_tiles)
    for e, row0, rows, _ in perm.tiles[:n].tolist():
        yield e, row0, rows


def moe_fp8_gemm_gate_up(xq, xs, w13, w13_scale, perm, status=None):
    inter = w13.shape[1] // 2
    hq = torch.zeros(xq.shape[0], inter, dtype=torch.uint8)
    hs = torch.zeros(xq.shape[0], inter // 128)
    for e, row0, rows in _rows_of_tiles(perm):
        a = moe_ref.dequant_act(xq[row0:row0 + rows].view(torch.float8_e4m3fn), xs[row0:row0 + rows])
        gu = a @ moe_ref.dequant_weight(w13[e].view(torch.float8_e4m3fn), w13_scale[e]).t()
        h = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
        q, s = moe_ref.act_quant_ref(h)
        hq[row0:row0 + rows], hs[row0:row0 + rows] = q.view(torch.uint8), s
    return hq, hs


def moe_fp8_gemm_down(hq, hs, w2, w2_scale, perm, status=None, out=None, out_row_map=None):
    y = out if out is not None else torch.zeros(hq.shape[0], w2.shape[1], dtype=torch.bfloat16)
    for e, row0, rows in _rows_of_tiles(perm):
        a = moe_ref.dequant_act(hq[row0:row0 + rows].view(torch.float8_e4m3fn), hs[row0:row0 + rows])
        val = (a @ moe_ref.dequant_weight(w2[e].view(torch.float8_e4m3fn), w2_scale[e]).t()).bfloat16()
        if out_row_map is None:
            y[row0:row0 + rows] = val
        else:
            y[out_row_map[row0:row0 + rows].long()] = val
    return y


def moe_combine(y, row_of_pair, w):
    T, K = w.shape
    rop = row_of_pair.long().view(T, K)
    out = torch.zeros(T, y.shape[1])
    for k in range(K):
        ok = (rop[:, k] >= 0).view(T, 1)  # a negative row (dropped pair) adds nothing
        out = out + torch.where(ok, w[:, k:k + 1] * y[rop[:, k].clamp(min=0)].float(), torch.zeros(1))
    return out.bfloat16()
