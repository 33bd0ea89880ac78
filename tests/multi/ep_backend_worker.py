"""Worker of tests/test_gpu_ep_multi.py: one process per GPU (torchrun).  Continuous batching over an
expert-parallel engine: every rank serves its OWN requests through B200Backend - different numbers of them, of
different lengths, at different times - while the MoE layers of all ranks exchange rows.  The ranks keep in
step through the backend's exchange rounds (a rank without work answers with idle passes).  Every request's
tokens must equal what a single-GPU engine holding all experts generates for it.  Prints "EP_BACKEND_OK <rank>"."""
import importlib
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
eng_mod = importlib.import_module("inference-server_b200.engine")
backend_mod = importlib.import_module("inference-server_b200.backend")


def sliced(layer, lo, hi):
    """The same layer holding only experts [lo, hi)."""
    w = eng_mod.LayerWeights()
    for name in eng_mod.LayerWeights.__slots__:
        setattr(w, name, getattr(layer, name))
    w.w13, w.w13_scale = layer.w13[lo:hi].contiguous(), layer.w13_scale[lo:hi].contiguous()
    w.w2, w.w2_scale = layer.w2[lo:hi].contiguous(), layer.w2_scale[lo:hi].contiguous()
    return w


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=dev)
    cfg = eng_mod.CONFIGS["tiny"]
    g = torch.Generator(device=dev).manual_seed(11)  # the same model on every rank
    full = [eng_mod.random_layer(cfg, dev, g) for _ in range(cfg.layers)]
    embed = (torch.randn(cfg.vocab_size, cfg.hidden, device=dev, generator=g) * 0.02).bfloat16()
    lm_head = (torch.randn(cfg.vocab_size, cfg.hidden, device=dev, generator=g) * 0.02).bfloat16()
    norm = torch.ones(cfg.hidden, device=dev, dtype=torch.bfloat16)
    el = cfg.experts // world
    common = dict(num_blocks=96, max_batch=32, max_pages_per_seq=8, device=dev, embed=embed, lm_head=lm_head,
                  final_norm=norm)
    ref_engine = eng_mod.DecodeEngine(cfg, layers=full, **common)
    ep_engine = eng_mod.DecodeEngine(cfg, layers=[sliced(w, rank * el, (rank + 1) * el) for w in full],
                                     ep_group=dist.group.WORLD, **common)
    assert ep_engine.ep_transport == "p2p", "peer-memory transport expected on one node"
    ref = backend_mod.B200Backend(ref_engine, max_new_tokens=24)
    be = backend_mod.B200Backend(ep_engine, max_new_tokens=24)
    be.enable_expert_parallel_rounds()

    # every rank has its own requests: rank 0 three, the others one, arriving at their own pace
    gp = torch.Generator().manual_seed(100 + rank)
    n_req = 3 if rank == 0 else 1
    reqs = [(torch.randint(0, cfg.vocab_size, (int(torch.randint(5, 30, (1,), generator=gp)),), generator=gp).tolist(),
             int(torch.randint(4, 20, (1,), generator=gp))) for _ in range(n_req)]
    if rank:
        time.sleep(0.3 * rank)  # joins while rank 0 is already decoding
    got = [be.generate(p, n) for p, n in reqs]
    # a batch of two with staggered lengths: admit, evict and a changing batch size under expert parallelism
    if rank == 0:
        got.append(be.generate_batch([reqs[0][0], reqs[1][0]], [reqs[0][1], reqs[1][1]]))
    store = dist.distributed_c10d._get_default_store()
    store.add("ep_backend_done", 1)
    while store.add("ep_backend_done", 0) < world:  # the others may still need this rank's experts
        time.sleep(0.01)
    time.sleep(0.1)
    rounds, idle = be._round_keeper.rounds, be._round_keeper.idle_rounds
    be.close()
    ep_engine.check_status(f"rank {rank}")

    want = [ref.generate(p, n) for p, n in reqs]
    if rank == 0:
        want.append(ref.generate_batch([reqs[0][0], reqs[1][0]], [reqs[0][1], reqs[1][1]]))
    assert got == want, f"rank {rank}: expert-parallel tokens {got} differ from the single-GPU engine's {want}"
    assert idle > 0 or world == 1 or rank == 0, f"rank {rank} never had to keep an exchange company ({rounds} rounds)"
    print(f"EP_BACKEND_OK {rank} rounds={rounds} idle={idle} tokens={sum(len(t) for t in got[:n_req])}", flush=True)
    dist.barrier()
    ep_engine._graphs.clear()
    ep_engine.ep_arena.close(importlib.import_module("inference-server_b200.ops"))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
