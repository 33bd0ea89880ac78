"""Expert-parallel dispatch/combine logic with two gloo ranks on CPU.

Each rank routes its own tokens, exchanges e4m3 rows through fixed-capacity all-to-alls, runs the experts it
owns (CPU stand-in kernels built from the oracle) and combines.  The result must equal the single-process
oracle layer on the same tokens with all experts local."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, capacity, results):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import importlib

    import oracle
    from oracle import cpu_kernels

    ep = importlib.import_module("inference-server_b200.ep")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E, K, H, I, T = 8, 2, 256, 128, 24
        g = torch.Generator().manual_seed(0)  # same weights on every rank
        w13q, w13s = oracle.quantize_weight_ref(torch.randn(E, 2 * I, H, generator=g) * 0.05)
        w2q, w2s = oracle.quantize_weight_ref(torch.randn(E, H, I, generator=g) * 0.05)
        gr = torch.Generator().manual_seed(100 + rank)  # different tokens per rank
        x = torch.randn(T, H, generator=gr).bfloat16()
        logits = torch.randn(T, E, generator=gr)
        el = E // world
        lo = rank * el
        st = ep.EPState(T, H, K, E, world, capacity, "cpu")
        out = ep.ep_moe_forward(
            st, x, logits, w13q[lo:lo + el].view(torch.uint8), w13s[lo:lo + el], w2q[lo:lo + el].view(torch.uint8),
            w2s[lo:lo + el], True, cpu_kernels, lambda o, i: dist.all_to_all_single(o, i))
        ref = oracle.moe_fp8_ref(x, logits, w13q, w13s, w2q, w2s, K, True)
        err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        results[rank] = (err, bool(st.overflow.item()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("capacity,expect_overflow", [(48, False), (16, True)])
def test_two_rank_expert_parallel_layer_matches_single_process(capacity, expect_overflow):
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29600 + (os.getpid() + capacity) % 300
    mp.spawn(_worker, args=(world, port, capacity, results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        err, overflow = results[rank]
        assert overflow == expect_overflow
        if not expect_overflow:
            assert err < 1e-2, f"rank {rank}: EP layer differs from the single-process layer by {err}"


def test_plan_dispatch_slots():
    sys.path.insert(0, ROOT)
    import importlib

    import oracle

    ep = importlib.import_module("inference-server_b200.ep")
    ids = torch.tensor([[0, 5], [4, 1], [7, 0], [6, 5]], dtype=torch.int32)
    p = oracle.permute_ref(ids, 8)
    slot, expert_of_slot, overflow = ep.plan_dispatch(ids, torch.from_numpy(p["row_of_pair"]),
                                                      torch.from_numpy(p["expert_offsets"]), 8, 2, 6)
    assert not bool(overflow)
    # rank 0 owns experts 0-3, rank 1 owns 4-7; within a destination rows are in expert-sorted order
    assert slot.tolist() == [0, 6 + 1, 6 + 0, 2, 6 + 4, 1, 6 + 3, 6 + 2]
    assert expert_of_slot.tolist() == [0, 0, 1, 4, 4, 4, 0, 1, 1, 2, 3, 4]
    assert ep.default_capacity(256, 8, 8) == 512
