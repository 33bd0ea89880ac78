"""The expert-parallel MoE layer's GPU path with a world of one (all-to-all = copy) vs the fused layer (B200).
Multi-rank slot logic is covered by tests/test_ep_gloo.py; this covers the same function on CUDA tensors with
the real kernels, including the local re-sort with empty slots."""
import pytest
import torch

from conftest import pkg, rel_err
import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("T,slack", [(64, 0), (64, 40), (256, 128)])
def test_ep_layer_world_one_matches_fused_layer(ops, T, slack):
    ep = pkg("ep")
    E, K, H, I = 128, 8, 2048, 768
    g = torch.Generator().manual_seed(T)
    w13q, w13s = oracle.quantize_weight_ref(torch.randn(E, 2 * I, H, generator=g) * 0.02)
    w2q, w2s = oracle.quantize_weight_ref(torch.randn(E, H, I, generator=g) * 0.02)
    dw = [w13q.view(torch.uint8).to(DEV), w13s.to(DEV), w2q.view(torch.uint8).to(DEV), w2s.to(DEV)]
    x = torch.randn(T, H, generator=g).bfloat16().to(DEV)
    logits = torch.randn(T, E, generator=g).bfloat16().to(DEV)
    ref = ops.moe_fp8_forward(x, logits, *dw, K, True)
    st = ep.EPState(T, H, K, E, 1, T * K + slack, DEV)  # slack leaves empty slots that must sort last and be skipped
    out = ep.ep_moe_forward(st, x, logits, *dw, True, ops, lambda o, i: o.copy_(i))
    torch.cuda.synchronize()
    assert not bool(st.overflow.item())
    assert rel_err(out, ref) < 1e-2
    assert torch.equal(out, ref)  # same rows, same order inside every expert: same bits
    # fused tail: residual add + next norm
    res1, res2 = x.clone(), x.clone()
    nw = torch.ones(H, dtype=torch.bfloat16, device=DEV)
    h1 = ops.moe_fp8_forward(x, logits, *dw, K, True, residual=res1, norm_weight=nw)
    h2 = ep.ep_moe_forward(st, x, logits, *dw, True, ops, lambda o, i: o.copy_(i), residual=res2, norm_weight=nw)
    assert torch.equal(res1, res2) and torch.equal(h1, h2)


def test_ep_layer_can_be_captured_in_a_cuda_graph(ops):
    """The decode step is replayed from a CUDA graph: the layer must not copy from the host or size anything
    by device data while it is being captured."""
    ep = pkg("ep")
    E, K, H, I, T = 128, 8, 2048, 768, 32
    g = torch.Generator().manual_seed(1)
    w13q, w13s = oracle.quantize_weight_ref(torch.randn(E, 2 * I, H, generator=g) * 0.02)
    w2q, w2s = oracle.quantize_weight_ref(torch.randn(E, H, I, generator=g) * 0.02)
    dw = [w13q.view(torch.uint8).to(DEV), w13s.to(DEV), w2q.view(torch.uint8).to(DEV), w2s.to(DEV)]
    x = torch.randn(T, H, generator=g).bfloat16().to(DEV)
    logits = torch.randn(T, E, generator=g).bfloat16().to(DEV)
    st = ep.EPState(T, H, K, E, 1, T * K + 16, DEV)
    run = lambda: ep.ep_moe_forward(st, x, logits, *dw, True, ops, lambda o, i: o.copy_(i))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ref = run().clone()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = run()
    x.copy_(torch.randn(T, H, generator=g).bfloat16())  # new input, replay must recompute
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, ops.moe_fp8_forward(x, logits, *dw, K, True))
    assert not torch.equal(out, ref)


@pytest.mark.parametrize("T,W,cap", [(64, 4, 256), (256, 8, 512), (64, 2, 200), (33, 4, 40)])
def test_dispatch_slot_kernel_matches_the_torch_plan(ops, T, W, cap):
    """b200_moe_permute_quant_ep places rows exactly where ep.plan_dispatch (plain torch index arithmetic,
    verified against the single-process layer by the gloo test) says, including the overflow case."""
    ep = pkg("ep")
    E, K, H = 128, 8, 2048
    g = torch.Generator().manual_seed(T + W)
    logits = torch.randn(T, E, generator=g)
    x = torch.randn(T, H, generator=g).bfloat16()
    ids, _ = oracle.route_ref(logits, K, True)
    r = oracle.permute_ref(ids, E)
    slot_ref, eos_ref, ovf_ref = ep.plan_dispatch(ids, torch.from_numpy(r["row_of_pair"]),
                                                  torch.from_numpy(r["expert_offsets"]), E, W, cap)
    xq_send = torch.zeros(W * cap, H, dtype=torch.uint8, device=DEV)
    xs_send = torch.zeros(W * cap, H // 128, dtype=torch.float32, device=DEV)
    eos = torch.full((W * cap,), -7, dtype=torch.int32, device=DEV)  # the kernel fills used AND empty slots
    ovf = torch.zeros(1, dtype=torch.int32, device=DEV)
    p, slot = ops.moe_permute_quant_ep(ids.to(DEV), x.to(DEV), E, W, cap, xq_send, xs_send, eos, ovf)
    ops.read_status(p.workspace, "moe_permute_quant_ep")
    assert torch.equal(slot.cpu().long(), slot_ref)
    assert torch.equal(eos.cpu(), eos_ref)
    assert bool(ovf.item()) == bool(ovf_ref)
    rq, rs = oracle.act_quant_ref(x)
    ok = slot_ref >= 0
    tok = torch.arange(T * K) // K
    assert torch.equal(xq_send.cpu()[slot_ref[ok]], rq.view(torch.uint8)[tok[ok]])
    assert torch.equal(xs_send.cpu()[slot_ref[ok]], rs[tok[ok]])
