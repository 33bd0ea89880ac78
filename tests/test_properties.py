"""Property tests (CPU, hypothesis) of the invariants the routing, permutation and dispatch code is held to.
They run on the oracle and on the package's torch-level host code; the GPU tests hold the kernels to the
oracle bit for bit, so the properties carry over."""
import importlib

import numpy as np
import torch
from hypothesis import given, settings, strategies as st

import oracle

ep = importlib.import_module("inference-server_b200.ep")
quant = importlib.import_module("inference-server_b200.quant")


@settings(max_examples=40, deadline=None)
@given(T=st.integers(1, 40), E=st.sampled_from([4, 16, 128]), K=st.integers(1, 4), seed=st.integers(0, 10**6),
       coarse=st.booleans())
def test_route_properties(T, E, K, seed, coarse):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if coarse:
        logits = (logits * 2).round() / 2  # many exact ties
    ids, w = oracle.route_ref(logits, K, True)
    assert ids.shape == (T, K) and ids.dtype == torch.int32
    for t in range(T):
        row = ids[t].tolist()
        assert len(set(row)) == K and all(0 <= e < E for e in row)  # distinct, in range
        vals = logits[t, ids[t].long()]
        assert torch.all(vals[:-1] >= vals[1:])  # value-descending
        for a, b in zip(range(K - 1), range(1, K)):
            if vals[a] == vals[b]:
                assert row[a] < row[b]  # ties: lower expert id first
        rest = torch.ones(E, dtype=torch.bool)
        rest[ids[t].long()] = False
        if rest.any():
            assert logits[t][rest].max() <= vals[-1]  # nothing better was left out
    np.testing.assert_allclose(w.sum(-1).numpy(), 1.0, rtol=1e-5)


@settings(max_examples=40, deadline=None)
@given(T=st.integers(0, 60), E=st.sampled_from([1, 3, 16, 130]), K=st.integers(1, 3), seed=st.integers(0, 10**6))
def test_permutation_properties(T, E, K, seed):
    rng = np.random.default_rng(seed)
    ids = torch.from_numpy(rng.integers(0, E, size=(T, K)).astype(np.int32))
    p = oracle.permute_ref(ids, E)
    n = T * K
    assert sorted(p["sorted_pair_ids"].tolist()) == list(range(n))  # a permutation
    assert np.array_equal(p["row_of_pair"][p["sorted_pair_ids"]], np.arange(n))  # inverse
    flat = ids.reshape(-1).numpy()
    es = flat[p["sorted_pair_ids"]]
    assert np.all(es[:-1] <= es[1:])  # grouped by expert
    for e in range(E):
        seg = p["sorted_pair_ids"][p["expert_offsets"][e]:p["expert_offsets"][e + 1]]
        assert np.all(flat[seg] == e) and np.all(seg[:-1] < seg[1:])  # stable inside an expert
    assert p["expert_offsets"][-1] == n
    covered = sum(int(r) for _, _, r, _ in p["tiles"].tolist())
    assert covered == n and all(0 < r <= 128 for _, _, r, _ in p["tiles"].tolist())


@settings(max_examples=40, deadline=None)
@given(T=st.integers(1, 50), K=st.integers(1, 4), W=st.sampled_from([1, 2, 4, 8]), cap=st.integers(1, 64),
       seed=st.integers(0, 10**6))
def test_dispatch_plan_properties(T, K, W, cap, seed):
    E = 16
    rng = np.random.default_rng(seed)
    ids = torch.from_numpy(np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32))
    p = oracle.permute_ref(ids, E)
    slot, eos, overflow = ep.plan_dispatch(ids, torch.from_numpy(p["row_of_pair"]),
                                           torch.from_numpy(p["expert_offsets"]), E, W, cap)
    el = E // W
    used = slot[slot >= 0]
    assert used.unique().numel() == used.numel()  # no two pairs share a slot
    flat = ids.reshape(-1).long()
    for pair in range(T * K):
        s = int(slot[pair])
        if s >= 0:
            assert s // cap == int(flat[pair]) // el  # the slot lies in the owner's segment
            assert int(eos[s]) == int(flat[pair]) % el  # and carries the owner-local expert id
    per_dst = torch.bincount(flat // el, minlength=W)
    assert bool(overflow) == bool((per_dst > cap).any())
    assert int((slot < 0).sum()) == int((per_dst - cap).clamp(min=0).sum())  # exactly the excess is dropped
    assert int((eos != el).sum()) == used.numel()  # every other slot is marked empty


@settings(max_examples=20, deadline=None)
@given(rows=st.integers(1, 3), cols=st.integers(1, 3), seed=st.integers(0, 10**6), zero=st.booleans())
def test_weight_quant_tile_round_trip(rows, cols, seed, zero):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(2, rows * 128, cols * 128, generator=g) * 0.05
    if zero:
        w[0, :128, :128] = 0
    q, s = quant.quantize_weight_blocks(w)
    q2, s2 = oracle.quantize_weight_ref(w)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)
    assert torch.equal(quant.untile_weight_blocks(quant.tile_weight_blocks(q.view(torch.uint8))), q.view(torch.uint8))
    back = quant.dequantize_weight_blocks(q, s)
    assert float((back - w).abs().max()) <= float(w.abs().max()) * 0.0715 + 1e-12  # half an e4m3 step of the tile maximum
