"""Worker of tests/test_gpu_ep_multi.py: one process per GPU (torchrun).  Every rank runs the expert-parallel
MoE layer on its own tokens with both transports (NCCL all-to-all, peer-memory stores) and compares each with
the single-GPU fused layer holding all experts.  Prints "EP_MULTI_OK <rank>" on success."""
import importlib
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
ops = importlib.import_module("inference-server_b200.ops")
ep = importlib.import_module("inference-server_b200.ep")
quant = importlib.import_module("inference-server_b200.quant")


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    E, K, H, I, T = 128, 8, 2048, 768, 64
    g = torch.Generator(device=dev).manual_seed(7)  # the same weights on every rank
    w13q, w13s = quant.quantize_weight_blocks(torch.randn(E, 2 * I, H, generator=g, device=dev) * 0.02)
    w2q, w2s = quant.quantize_weight_blocks(torch.randn(E, H, I, generator=g, device=dev) * 0.02)
    El = E // world
    local = [t[rank * El:(rank + 1) * El].contiguous() for t in (w13q, w13s, w2q, w2s)]
    gt = torch.Generator(device=dev).manual_seed(100 + rank)  # different tokens on every rank
    cap = ep.default_capacity(T, K, world)
    a2a = lambda o, i: dist.all_to_all_single(o, i)
    st_nccl = ep.EPState(T, H, K, E, world, cap, dev)
    arena = ep.PeerArena(H, world, cap, dev)
    arena.connect(ops, dist.group.WORLD)
    st_p2p = ep.EPState(T, H, K, E, world, cap, dev, arena=arena)
    for it in range(3):
        x = torch.randn(T, H, generator=gt, device=dev).bfloat16()
        logits = torch.randn(T, E, generator=gt, device=dev).bfloat16()
        ref = ops.moe_fp8_forward(x, logits, w13q, w13s, w2q, w2s, K, True)
        out_nccl = ep.ep_moe_forward(st_nccl, x, logits, *local, True, ops, a2a)
        out_p2p = ep.ep_moe_forward(st_p2p, x, logits, *local, True, ops, None)
        torch.cuda.synchronize()
        ops.read_status(st_p2p.status, "peer-memory exchange")
        assert not bool(st_nccl.overflow.item()) and not bool(st_p2p.overflow.item())
        assert torch.equal(out_nccl, ref), f"rank {rank} pass {it}: NCCL transport differs from the fused layer"
        assert torch.equal(out_p2p, ref), f"rank {rank} pass {it}: peer-memory transport differs from the fused layer"
    assert st_p2p.epochs.tolist() == [3, 3]
    # the same layer inside a CUDA graph, replayed on new inputs
    x = torch.randn(T, H, generator=gt, device=dev).bfloat16()
    logits = torch.randn(T, E, generator=gt, device=dev).bfloat16()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ep.ep_moe_forward(st_p2p, x, logits, *local, True, ops, None)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = ep.ep_moe_forward(st_p2p, x, logits, *local, True, ops, None)
    for it in range(3):
        x.copy_(torch.randn(T, H, generator=gt, device=dev).bfloat16())
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, ops.moe_fp8_forward(x, logits, w13q, w13s, w2q, w2s, K, True)), f"rank {rank} replay {it}"
    ops.read_status(st_p2p.status, "peer-memory exchange (graph)")
    print(f"EP_MULTI_OK {rank}", flush=True)
    del graph
    torch.cuda.synchronize()
    dist.barrier()
    arena.close(ops)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
