"""Expert parallelism over peer memory on ONE GPU (B200): the dispatch kernel and the down-GEMM epilogue store
rows into "peer" receive buffers, flag exchanges order the stages.

Several ranks are emulated in one process: every rank has its own tokens, arena and expert slice, the peers'
arenas are plain device pointers, and the layer runs stage by stage over all ranks with ep_signal / ep_wait
apart (kernels that wait for each other must not be queued behind one another).  What this cannot cover -
CUDA IPC mapping and visibility across GPUs - is covered by tests/test_gpu_ep_multi.py on a box with two GPUs.
"""
import pytest
import torch

from conftest import pkg, rel_err
import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
E, K, H, I = 128, 8, 2048, 768


def layer_weights(seed):
    g = torch.Generator().manual_seed(seed)
    w13q, w13s = oracle.quantize_weight_ref(torch.randn(E, 2 * I, H, generator=g) * 0.02)
    w2q, w2s = oracle.quantize_weight_ref(torch.randn(E, H, I, generator=g) * 0.02)
    return [w13q.view(torch.uint8).to(DEV), w13s.to(DEV), w2q.view(torch.uint8).to(DEV), w2s.to(DEV)]


@pytest.mark.parametrize("T,slack", [(64, 0), (256, 128)])
def test_world_of_one_with_an_arena_matches_the_fused_layer(ops, T, slack):
    ep = pkg("ep")
    dw = layer_weights(T)
    g = torch.Generator().manual_seed(T + 1)
    x = torch.randn(T, H, generator=g).bfloat16().to(DEV)
    logits = torch.randn(T, E, generator=g).bfloat16().to(DEV)
    ref = ops.moe_fp8_forward(x, logits, *dw, K, True)
    cap = T * K + slack
    arena = ep.PeerArena(H, 1, cap, DEV)
    st = ep.EPState(T, H, K, E, 1, cap, DEV, arena=arena)
    for _ in range(2):  # twice: the epochs advance and the buffers are reused
        out = ep.ep_moe_forward(st, x, logits, *dw, True, ops, None)
        torch.cuda.synchronize()
        ops.read_status(st.status, "ep p2p")
        assert not bool(st.overflow.item())
        assert torch.equal(out, ref)
    assert st.epochs.tolist() == [2, 2]


@pytest.mark.parametrize("W,T,cap", [(2, 64, 512), (4, 64, 256), (8, 32, 64)])
def test_emulated_ranks_match_the_single_gpu_layer(ops, W, T, cap):
    """Every emulated rank must get, for its own tokens, exactly what the whole-model layer gives: a row's
    result does not depend on which other rows share its expert's tile."""
    ep = pkg("ep")
    dw = layer_weights(W)
    El = E // W
    local = [[dw[0][r * El:(r + 1) * El].contiguous(), dw[1][r * El:(r + 1) * El].contiguous(),
              dw[2][r * El:(r + 1) * El].contiguous(), dw[3][r * El:(r + 1) * El].contiguous()] for r in range(W)]
    g = torch.Generator().manual_seed(100 + W)
    xs = [torch.randn(T, H, generator=g).bfloat16().to(DEV) for _ in range(W)]
    lg = [torch.randn(T, E, generator=g).bfloat16().to(DEV) for _ in range(W)]
    arenas = [ep.PeerArena(H, W, cap, DEV) for _ in range(W)]
    for r, a in enumerate(arenas):
        a.connect_in_process(arenas, r)
    states = [ep.EPState(T, H, K, E, W, cap, DEV, arena=arenas[r]) for r in range(W)]
    for rep in range(2):
        sent = [ep.p2p_dispatch(states[r], xs[r], lg[r], True, ops) for r in range(W)]
        for r in range(W):
            ops.ep_signal(states[r].peer_flags[0], states[r].epochs[0:1], r, W)
        for r in range(W):
            ops.ep_wait(states[r].flags[0], states[r].epochs[0:1], W, states[r].status)
            ep.p2p_experts(states[r], *local[r], ops)
            ops.ep_signal(states[r].peer_flags[1], states[r].epochs[1:2], r, W)
        outs = []
        for r in range(W):
            ops.ep_wait(states[r].flags[1], states[r].epochs[1:2], W, states[r].status)
            outs.append(ep._combine(states[r], sent[r][0], sent[r][1], ops, None, None, 1e-6))
        torch.cuda.synchronize()
        for r in range(W):
            ops.read_status(states[r].status, f"rank {r}")
            assert not bool(states[r].overflow.item())
            ref = ops.moe_fp8_forward(xs[r], lg[r], *dw, K, True)
            assert rel_err(outs[r], ref) < 1e-2
            assert torch.equal(outs[r], ref), f"rank {r}, pass {rep}"
            assert states[r].flags[0].tolist()[:W] == [rep + 1] * W


def test_a_wait_nobody_answers_runs_out_and_reports(ops):
    """A bounded wait: a flag that nothing sets.  The kernel gives up after about a second, records the
    peer-timeout code in the status word and the stream carries on."""
    flags = torch.zeros(8, dtype=torch.int32, device=DEV)
    epoch = torch.ones(1, dtype=torch.int32, device=DEV)
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    ops.ep_wait(flags, epoch, 2, status)
    after = torch.ones(4, device=DEV) * 2  # the stream is still usable
    torch.cuda.synchronize()
    assert after.sum().item() == 8
    with pytest.raises(Exception, match="rank's flag"):
        ops.read_status(status, "ep_wait")


@pytest.mark.parametrize("n,El,H_", [(4096, 16, 2048), (512, 32, 2048), (300, 4, 512)])
def test_fused_receive_side_sort_and_copy(ops, n, El, H_):
    """b200_moe_permute_gather_fp8 = b200_moe_permute (with the dummy expert El for empty slots) followed by
    b200_gather_rows_fp8, except that rows of the dummy expert are not copied."""
    g = torch.Generator().manual_seed(n)
    ids = torch.randint(0, El + 1, (n,), generator=g, dtype=torch.int32).to(DEV)
    src_q = torch.randint(0, 256, (n, H_), generator=g, dtype=torch.uint8).to(DEV)
    src_s = torch.rand(n, H_ // 128, generator=g).to(DEV)
    ref = ops.moe_permute(ids.view(-1, 1), El + 1, El)
    rq, rs = ops.gather_rows_fp8(src_q, src_s, ref.sorted_pair_ids)
    dq = torch.full((n, H_), 0xAB, dtype=torch.uint8, device=DEV)
    ds = torch.full((n, H_ // 128), -1.0, device=DEV)
    p = ops.moe_permute_gather_fp8(ids, El + 1, El, src_q, src_s, dq, ds)
    torch.cuda.synchronize()
    ops.read_status(p.workspace, "moe_permute_gather_fp8")
    assert torch.equal(p.sorted_pair_ids, ref.sorted_pair_ids) and torch.equal(p.row_of_pair, ref.row_of_pair)
    assert torch.equal(p.expert_offsets, ref.expert_offsets) and int(p.num_tiles) == int(ref.num_tiles)
    nt = int(ref.num_tiles)
    assert torch.equal(p.tiles[:nt], ref.tiles[:nt])
    real = int(ref.expert_offsets[El])  # rows of real experts come first
    assert torch.equal(dq[:real], rq[:real]) and torch.equal(ds[:real], rs[:real])
    assert bool((dq[real:] == 0xAB).all()) and bool((ds[real:] == -1.0).all())


def test_combine_skips_negative_rows(ops):
    T, K_, H_ = 16, 4, 512
    g = torch.Generator().manual_seed(3)
    y = torch.randn(T * K_, H_, generator=g).bfloat16().to(DEV)
    w = torch.rand(T, K_, generator=g).to(DEV)
    rows = torch.randperm(T * K_, generator=g).to(torch.int32).to(DEV)
    drop = torch.rand(T * K_, generator=g).to(DEV) < 0.3
    ref = ops.moe_combine(y, rows, torch.where(drop.view(T, K_), torch.zeros_like(w), w))
    out = ops.moe_combine(y, torch.where(drop, torch.full_like(rows, -1), rows), w)
    assert torch.equal(out, ref)
    x1 = torch.randn(T, H_, generator=g).bfloat16().to(DEV)
    x2 = x1.clone()
    nw = torch.rand(H_, generator=g).bfloat16().to(DEV)
    h1 = ops.moe_combine_add_rmsnorm(y, rows, torch.where(drop.view(T, K_), torch.zeros_like(w), w), x1, nw, 1e-6)
    h2 = ops.moe_combine_add_rmsnorm(y, torch.where(drop, torch.full_like(rows, -1), rows), w, x2, nw, 1e-6)
    assert torch.equal(h1, h2) and torch.equal(x1, x2)
