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


def _worker(rank, world, port, capacity, results, valid_rows=None):
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
        n = T if valid_rows is None else valid_rows[rank]  # real rows of this rank's pass; the rest is padding
        out = ep.ep_moe_forward(
            st, x, logits, w13q[lo:lo + el].view(torch.uint8), w13s[lo:lo + el], w2q[lo:lo + el].view(torch.uint8),
            w2s[lo:lo + el], True, cpu_kernels, lambda o, i: dist.all_to_all_single(o, i),
            n_valid=None if valid_rows is None else torch.tensor([n], dtype=torch.int32))
        err = 0.0
        if n:
            ref = oracle.moe_fp8_ref(x[:n], logits[:n], w13q, w13s, w2q, w2s, K, True)
            err = float((out[:n].float() - ref.float()).abs().max() / ref.float().abs().max())
        pad_is_zero = bool((out[n:] == 0).all())
        results[rank] = (err, bool(st.overflow.item()), pad_is_zero)
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
        err, overflow, _ = results[rank]
        assert overflow == expect_overflow
        if not expect_overflow:
            assert err < 1e-2, f"rank {rank}: EP layer differs from the single-process layer by {err}"


@pytest.mark.parametrize("valid_rows", [(24, 5), (0, 17), (0, 0)])
def test_ranks_with_unequal_batches_share_one_fixed_shape_exchange(valid_rows):
    """Continuous batching gives every rank its own batch size; the exchange keeps one shape and the rows a
    rank does not have are padding that is routed nowhere.  A rank with no rows at all still serves its
    experts to the other."""
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29300 + (os.getpid() + sum(valid_rows) * 7) % 250
    mp.spawn(_worker, args=(world, port, 48, results, valid_rows), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        err, overflow, pad_is_zero = results[rank]
        assert not overflow and pad_is_zero
        assert err < 1e-2, f"rank {rank}: {valid_rows[rank]} real rows differ from the single-process layer by {err}"


def _round_worker(rank, world, port, passes, results):
    """Every rank has its own number of passes with work, arriving at its own pace; a pass is a collective
    (as an exchange is), so a rank that ran one more or one fewer than the others would hang the group."""
    sys.path.insert(0, ROOT)
    import importlib
    import threading
    import time

    ep = importlib.import_module("inference-server_b200.ep")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        gate = ep.RoundGate()
        log = []

        def one_pass(kind):
            t = torch.tensor([1 if kind == "work" else 0])
            dist.all_reduce(t)  # stands in for the layer exchanges of one pass
            log.append((kind, int(t)))

        lock = threading.Lock()
        keeper = ep.RoundKeeper(gate, lambda: one_pass("idle"), lock, idle_sleep=0.001).start()
        for i in range(passes[rank]):
            time.sleep(0.003 * (rank + 1))  # requests arrive between ticks
            with lock:  # as the scheduler holds the backend lock for a tick
                keeper.work_round()
                one_pass("work")
        # wait (on the host, without a collective: the keeper thread owns those) until every rank has done its
        # own work; the keeper meanwhile answers the rounds the slower ranks still start
        results[("done", rank)] = True
        while not all(results.get(("done", r)) for r in range(world)):
            time.sleep(0.01)
        time.sleep(0.05)
        with lock:
            rounds, idle = keeper.rounds, keeper.idle_rounds
        keeper.close()
        # a rank that is told a peer has left refuses further rounds instead of waiting for it
        refused = False
        try:
            keeper.work_round()
        except RuntimeError:
            refused = True
        results[rank] = (rounds, idle, sum(1 for k, _ in log if k == "work"), refused)
    finally:
        dist.destroy_process_group()


def test_round_keeper_keeps_ranks_in_step_with_unequal_work():
    world, passes = 2, (7, 2)
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29700 + os.getpid() % 150
    mp.spawn(_round_worker, args=(world, port, passes, results), nprocs=world, join=True)
    rounds = [results[r][0] for r in range(world)]
    assert rounds[0] == rounds[1], "ranks ran different numbers of exchange passes"
    assert max(passes) <= rounds[0] <= sum(passes)
    for r in range(world):
        total, idle, worked, refused = results[r]
        assert worked == passes[r] and idle == total - worked and refused


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


# ------------------------------------------------------------ peer arena ----
class _FakeIpc:
    """Stand-in for the ops IPC calls: handles are (rank, address) pairs, importing one "maps" it to a fake
    address; optionally one rank fails to export or to import."""

    def __init__(self, rank, fail_export_on=None, fail_import_on=None):
        self.rank, self.fail_export_on, self.fail_import_on = rank, fail_export_on, fail_import_on
        self.closed = []

    def ipc_export(self, t):
        if self.rank == self.fail_export_on:
            raise RuntimeError("export refused")
        return (b"H%03d" % self.rank).ljust(64, b"\0"), 128

    def ipc_import(self, handle, offset):
        if self.rank == self.fail_import_on:
            raise RuntimeError("import refused")
        peer = int(handle[1:4])
        return 1_000_000 * (peer + 1), 1_000_000 * (peer + 1) + offset

    def ipc_close(self, base):
        self.closed.append(base)


def _arena_worker(rank, world, port, fail_export_on, fail_import_on, results):
    sys.path.insert(0, ROOT)
    import importlib

    ep = importlib.import_module("inference-server_b200.ep")
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        arena = ep.PeerArena(256, world, 32, "cpu")
        fake = _FakeIpc(rank, fail_export_on, fail_import_on)
        ok = arena.connect(fake, dist.group.WORLD)
        results[rank] = (ok, list(arena.bases), list(fake.closed), list(arena.failures), arena.buf.data_ptr())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fail_export_on,fail_import_on", [(None, None), (1, None), (None, 0)])
def test_peer_arena_connect_agrees_on_every_rank(fail_export_on, fail_import_on):
    """The mapping either succeeds on every rank or every rank alike falls back (and unmaps what it had):
    a rank must never be left waiting in a collective for one that gave up."""
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29900 + (os.getpid() * 3 + (fail_export_on or 0) * 2 + (fail_import_on is not None)) % 90
    mp.spawn(_arena_worker, args=(world, port, fail_export_on, fail_import_on, results), nprocs=world, join=True)
    assert len(results) == world
    oks = [results[r][0] for r in range(world)]
    assert oks == [fail_export_on is None and fail_import_on is None] * world
    for rank in range(world):
        ok, bases, closed, failures, own = results[rank]
        if ok:
            other = 1 - rank
            assert bases[rank] == own and bases[other] == 1_000_000 * (other + 1) + 128
            assert closed == [] and failures == []
        else:
            assert bases == [own]
            assert failures and "refused" in failures[0]
            # a rank that had mapped its peer before the other one failed has unmapped it again
            assert len(closed) <= 1


def test_peer_arena_layout_is_aligned_and_disjoint():
    sys.path.insert(0, ROOT)
    import importlib

    ep = importlib.import_module("inference-server_b200.ep")
    for hidden, world, cap in [(2048, 8, 512), (4096, 4, 48), (512, 2, 16)]:
        a = ep.PeerArena(hidden, world, cap, "cpu")
        rows = world * cap
        offs = [a.off_xq, a.off_xs, a.off_id, a.off_y, a.off_flags, a.nbytes]
        sizes = [rows * hidden, rows * (hidden // 128) * 4, rows * 4, rows * hidden * 2, 64]
        assert all(o % 256 == 0 for o in offs[:-1])
        for o, n, nxt in zip(offs, sizes, offs[1:]):
            assert o + n <= nxt
        st = ep.EPState(4, hidden, 2, 8 * world, world, cap, "cpu", arena=a)
        assert st.xq_recv.shape == (rows, hidden) and st.y_recv.dtype == torch.bfloat16
        assert st.flags[0].numel() == 8 and st.flags[1].data_ptr() - st.flags[0].data_ptr() == 32
        assert st.peer_flags[1][0] == a.buf.data_ptr() + a.off_flags + 32
