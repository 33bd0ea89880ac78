"""Per-kernel microbenchmarks of the decode path on one B200 (synthetic, seeded inputs).

    python microbench.py attn            # paged decode attention, 64 sequences,
                                                               # contexts U{512..8192}, groups of 8 share 1024 tokens
    python microbench.py moe             # FP8 MoE layer, T in {1,16,64,256,1024,4096}
    python microbench.py ep --world 8    # expert-parallel layer, ranks emulated in-process
    python microbench.py fp8peak         # dense e4m3 GEMM rate of the library (cuBLASLt),
                                                               # the denominator for the MoE GEMM's tensor fraction
    python microbench.py prefill         # tiled causal prompt attention: a chunk of 1024 tokens at several
                                                               # depths of one sequence, beside the row-per-token form
    python microbench.py dense           # the bf16 projections (q/k/v, o, router, lm_head + arg-max) at decode
                                                               # sizes, every K split, beside the library GEMM
    ... attn --small / moe --small                             # few launches on a few hundred MB: sized for a profiler

Every case prints one JSON line per measured point: CUDA-event time (median of --iters launches after 3 warm-ups,
a 256 MB buffer written between launches so nothing stays in the 126 MB L2), the algorithmic bytes or flops of
the launch and the achieved rate.  It sits beside bench.py, outside the package, and only calls the package's `ops`.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
ops = importlib.import_module("inference-server_b200.ops")
quant = importlib.import_module("inference-server_b200.quant")
ep = importlib.import_module("inference-server_b200.ep")
DEV = "cuda"
PAGE = 16
MOE_TOKENS_DEFAULT = "1,16,64,256,1024,4096"


def measured_hbm_gbs() -> tuple[float, str]:
    """HBM copy bandwidth measured on this pool if the file is there, else the fallback figure."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class Timer:
    def __init__(self, iters: int, flush: bool = True):
        self.iters = iters
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV) if flush else None

    def __call__(self, fn, warm: int = 3) -> tuple[float, float]:
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(self.iters):
            if self.flush is not None:
                self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return float(np.median(ts)), float(np.min(ts))


# ------------------------------------------------------------------ attention --
def paged_case(batch, hq, hkv, d, ctx_lens, seed, group=0, shared_tokens=0):
    """Seeded page pools and a shuffled block table; rows of a group reuse the pages of their first
    `shared_tokens` tokens (full pages only), like radix prefix hits.  Returns device tensors and the number of
    distinct pages the batch reads."""
    rng = np.random.default_rng(seed)
    n_pages = [(L + PAGE - 1) // PAGE for L in ctx_lens]
    total = sum(n_pages) + 8
    perm = rng.permutation(total).tolist()
    table = np.zeros((batch, max(n_pages)), dtype=np.int32)
    shared: dict = {}
    for b, L in enumerate(ctx_lens):
        for p in range(n_pages[b]):
            if group and (p + 1) * PAGE <= min(L, shared_tokens):
                key = (b // group, p)
                if key not in shared:
                    shared[key] = perm.pop()
                table[b, p] = shared[key]
            else:
                table[b, p] = perm.pop()
    g = torch.Generator(device=DEV).manual_seed(seed)
    k_pool = torch.randn(total, hkv, PAGE, d, generator=g, device=DEV).bfloat16()
    v_pool = torch.randn(total, hkv, PAGE, d, generator=g, device=DEV).bfloat16()
    q = torch.randn(batch, hq, d, generator=g, device=DEV).bfloat16()
    unique = len({int(table[b, p]) for b in range(batch) for p in range(n_pages[b])})
    return q, k_pool, v_pool, torch.from_numpy(table).to(DEV), torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), unique


def run_attn(args) -> None:
    hq, hkv, d = args.q_heads, args.kv_heads, args.head_dim
    if args.small:
        batch, lens, group, shared = 16, [4096] * 16, 0, 0
    else:
        batch = args.batch
        lens = np.random.default_rng(0).integers(args.ctx_min, args.ctx_max + 1, size=batch).tolist()
        group, shared = args.share_group, args.share_tokens
    q, kp, vp, table, ctx, unique = paged_case(batch, hq, hkv, d, lens, 0, group, shared)
    alg = unique * PAGE * hkv * d * 2 * 2 + batch * hq * d * 2 * 2 + 4 * sum((L + PAGE - 1) // PAGE for L in lens) + 4 * batch
    st = args.split_tokens or ops.default_split_tokens(batch, hkv, table.shape[1] * PAGE)
    ws = ops.paged_attn_workspace(batch, hq, d, table.shape[1], PAGE, st, DEV)
    out = torch.empty_like(q)
    fn = lambda: ops.paged_attn_decode(q, kp, vp, table, ctx, d ** -0.5, st, ws, out)
    if args.small:
        for _ in range(4):
            fn()
        torch.cuda.synchronize()
        ops.read_status(ws, "attention")
        print(json.dumps({"case": "attn --small", "launches": 4, "alg_MB": alg / 1e6, "split_tokens": st}))
        return
    med, mn = Timer(args.iters)(fn)
    ops.read_status(ws, "attention")
    peak, src = measured_hbm_gbs()
    print(json.dumps({"case": "attn", "batch": batch, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
                      "mean_ctx": float(np.mean(lens)), "split_tokens": st, "us_median": med, "us_min": mn,
                      "alg_MB": alg / 1e6, "logical_MB": sum(lens) * hkv * d * 4 / 1e6, "GBs": alg / med / 1e3,
                      "frac_of_hbm_peak": alg / med / 1e3 / peak, "peak_GBs": peak, "peak_source": src,
                      "note": "time covers the split kernel and the split reduce"}))


# ------------------------------------------------------------------------ MoE --
def moe_weights(E, H, I, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    w13q, w13s = quant.quantize_weight_blocks(torch.randn(E, 2 * I, H, generator=g, device=DEV) * 0.02)
    w2q, w2s = quant.quantize_weight_blocks(torch.randn(E, H, I, generator=g, device=DEV) * 0.02)
    return w13q, w13s, w2q, w2s


def run_moe(args) -> None:
    E, K, H, I = args.experts, args.top_k, args.hidden, args.inter
    w13q, w13s, w2q, w2s = moe_weights(E, H, I)
    if args.tiled:  # the same values re-ordered into contiguous 128x128 blocks (bit-identical results)
        w13q = quant.tile_weight_blocks(w13q.view(torch.uint8))
        w2q = quant.tile_weight_blocks(w2q.view(torch.uint8))
    g = torch.Generator(device=DEV).manual_seed(1)
    tokens = [int(t) for t in args.tokens.split(",")]
    if args.small:
        tokens = tokens[:1] if args.tokens != MOE_TOKENS_DEFAULT else [64]
    timer = Timer(args.iters)
    peak, src = measured_hbm_gbs()
    for T in tokens:
        x = torch.randn(T, H, generator=g, device=DEV).bfloat16()
        logits = torch.randn(T, E, generator=g, device=DEV)
        ws = ops.moe_fp8_workspace(T, E, K, H, I, DEV)
        out = torch.empty_like(x)
        layer = lambda: ops.moe_fp8_forward(x, logits, w13q, w13s, w2q, w2s, K, True, ws, out)
        if args.small:
            for _ in range(3):
                layer()
            torch.cuda.synchronize()
            ops.read_status(ws, "moe")
            print(json.dumps({"case": "moe --small", "tokens": T, "launches_of_each_kernel": 3}))
            return
        med, mn = timer(layer)
        ids, _ = ops.moe_route(logits, K)
        hit = int(torch.unique(ids).numel())
        p = ops.moe_permute(ids, E)
        xq, xs = ops.act_quant_fp8(x, p.row_of_pair, K)
        status = torch.zeros(64, dtype=torch.int32, device=DEV)
        hq, hs = ops.moe_fp8_gemm_gate_up(xq, xs, w13q, w13s, p, status)
        gu, _ = timer(lambda: ops.moe_fp8_gemm_gate_up(xq, xs, w13q, w13s, p, status))
        dn, _ = timer(lambda: ops.moe_fp8_gemm_down(hq, hs, w2q, w2s, p, status))
        ops.read_status(status, "moe gemm")
        ops.read_status(ws, "moe")
        scale_bytes = 3 * H * I // 16384 * 4
        wbytes = hit * (3 * H * I + scale_bytes)
        alg = wbytes + T * H * 4 + T * E * 4
        flops = T * K * 6 * H * I
        print(json.dumps({"case": "moe", "tokens": T, "tiled_weights": bool(args.tiled), "experts_hit": hit, "layer_us_median": med, "layer_us_min": mn,
                          "gate_up_us": gu, "down_us": dn, "alg_MB": alg / 1e6, "layer_GBs": alg / med / 1e3,
                          "gate_up_GBs": hit * 2 * H * I / gu / 1e3, "down_GBs": hit * H * I / dn / 1e3,
                          "frac_of_hbm_peak_gemms": wbytes / (gu + dn) / 1e3 / peak, "layer_TFLOPs": flops / med / 1e6,
                          "gemm_TFLOPs": flops / (gu + dn) / 1e6, "peak_GBs": peak, "peak_source": src}))


# -------------------------------------------------------- expert parallelism --
def run_ep(args) -> None:
    """The peer-memory expert-parallel layer with `--world` ranks emulated in this process: every rank has its
    own tokens, arena and expert slice; the peers' arenas are plain device pointers.  The layer runs stage by
    stage over all ranks with signal and wait apart (launches that wait for each other must not queue behind
    one another on one GPU).  Prints the time of one whole pass over all ranks divided by the rank count."""
    W, T = args.world, args.tokens_per_rank
    E, K, H, I = args.experts, args.top_k, args.hidden, args.inter
    El = E // W
    w13q, w13s, w2q, w2s = moe_weights(El, H, I)  # the same slice stands in for every rank's experts
    cap = ep.default_capacity(T, K, W)
    arenas = [ep.PeerArena(H, W, cap, DEV) for _ in range(W)]
    for r, a in enumerate(arenas):
        a.connect_in_process(arenas, r)
    sts = [ep.EPState(T, H, K, E, W, cap, DEV, arena=arenas[r]) for r in range(W)]
    g = torch.Generator(device=DEV).manual_seed(2)
    xs = [torch.randn(T, H, generator=g, device=DEV).bfloat16() for _ in range(W)]
    lg = [torch.randn(T, E, generator=g, device=DEV).bfloat16() for _ in range(W)]
    res = [torch.zeros(T, H, dtype=torch.bfloat16, device=DEV) for _ in range(W)]
    nw = torch.ones(H, dtype=torch.bfloat16, device=DEV)

    def one_pass():
        sent = [ep.p2p_dispatch(sts[r], xs[r], lg[r], True, ops) for r in range(W)]
        for r in range(W):
            ops.ep_signal(sts[r].peer_flags[0], sts[r].epochs[0:1], r, W)
        for r in range(W):
            ops.ep_wait(sts[r].flags[0], sts[r].epochs[0:1], W, sts[r].status)
            ep.p2p_experts(sts[r], w13q, w13s, w2q, w2s, ops)
            ops.ep_signal(sts[r].peer_flags[1], sts[r].epochs[1:2], r, W)
        for r in range(W):
            ops.ep_wait(sts[r].flags[1], sts[r].epochs[1:2], W, sts[r].status)
            ep._combine(sts[r], sent[r][0], sent[r][1], ops, res[r], nw, 1e-6)

    for _ in range(2):
        one_pass()
    torch.cuda.synchronize()
    if args.small:
        for st in sts:
            ops.read_status(st.status, "ep")
        print(json.dumps({"case": "ep --small", "world": W, "passes": 2, "capacity": cap}))
        return
    graph = torch.cuda.CUDAGraph()  # replayed from a graph so that host launch time does not count
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph):
            one_pass()
    torch.cuda.current_stream().wait_stream(side)
    med, mn = Timer(args.iters, flush=False)(graph.replay)
    for st in sts:
        ops.read_status(st.status, "ep")
        assert not bool(st.overflow.item())
    print(json.dumps({"case": "ep", "world": W, "tokens_per_rank": T, "capacity": cap, "local_experts": El,
                      "us_per_rank_layer_median": med / W, "us_per_rank_layer_min": mn / W,
                      "note": "all ranks on one GPU: no NVLink time and no waiting for other ranks"}))


# ----------------------------------------------------------- prompt attention --
def run_prefill(args) -> None:
    """b200_paged_attn_prefill on a chunk of `--chunk` consecutive prompt tokens whose sequence already holds
    `first` tokens, for several `first`; flops = 4 * Hq * D * unmasked (query, key) pairs.  Beside it the decode
    kernel's row-per-token form (two rows per CTA) on the same rows."""
    hq, hkv, d, chunk = args.q_heads, args.kv_heads, args.head_dim, args.chunk
    firsts = [int(f) for f in args.first.split(",")]
    total = max(firsts) + chunk
    n_pages = (total + PAGE - 1) // PAGE
    g = torch.Generator(device=DEV).manual_seed(0)
    kp = torch.randn(n_pages + 8, hkv, PAGE, d, generator=g, device=DEV).bfloat16()
    vp = torch.randn(n_pages + 8, hkv, PAGE, d, generator=g, device=DEV).bfloat16()
    q = torch.randn(chunk, hq, d, generator=g, device=DEV).bfloat16()
    row = torch.randperm(n_pages + 8, generator=torch.Generator().manual_seed(0))[:n_pages].to(torch.int32).to(DEV)
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    if args.small:
        for _ in range(3):
            ops.paged_attn_prefill(q, kp, vp, row, firsts[0], d ** -0.5, status, out)
        torch.cuda.synchronize()
        ops.read_status(status, "prefill attention")
        print(json.dumps({"case": "prefill --small", "launches": 3, "chunk": chunk, "first_position": firsts[0]}))
        return
    timer = Timer(args.iters)
    table = row.view(1, -1).expand(chunk, -1).contiguous()
    for first in firsts:
        med, mn = timer(lambda: ops.paged_attn_prefill(q, kp, vp, row, first, d ** -0.5, status, out))
        pairs = chunk * first + chunk * (chunk + 1) // 2
        flops = 4 * hq * d * pairs
        lens = torch.arange(first + 1, first + chunk + 1, dtype=torch.int32, device=DEV)
        st = ops.default_split_tokens(chunk, hkv, table.shape[1] * PAGE)
        ws = ops.paged_attn_workspace(chunk, hq, d, table.shape[1], PAGE, st, DEV)
        rows_med, _ = timer(lambda: ops.paged_attn_decode(q, kp, vp, table, lens, d ** -0.5, st, ws, out, pairs=True))
        print(json.dumps({"case": "prefill", "chunk": chunk, "first_position": first, "q_heads": hq, "kv_heads": hkv,
                          "us_median": med, "us_min": mn, "GFLOP": flops / 1e9, "TFLOPs": flops / med / 1e6,
                          "row_per_token_form_us": rows_med}))
    ops.read_status(status, "prefill attention")


# --------------------------------------------------------- dense projections --
def run_dense(args) -> None:
    """The step's bf16 projections at `--rows` rows: this package's tcgen05 kernel for every K split it offers,
    and torch.matmul (cuBLAS) on the same tensors for comparison.  Bytes = the weight matrix once."""
    M, H = args.rows, args.hidden
    qkv_out = (args.q_heads + 2 * args.kv_heads) * args.head_dim
    shapes = [("qkv", qkv_out, H), ("o", H, args.q_heads * args.head_dim), ("router", args.experts, H)]
    g = torch.Generator(device=DEV).manual_seed(0)
    timer = Timer(args.iters)
    peak, src = measured_hbm_gbs()
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    for name, N, K in shapes:
        x = torch.randn(M, K, generator=g, device=DEV).bfloat16()
        w = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        gws = ops.dense_gemm_workspace(M, N, DEV)
        row = {"case": "dense", "what": name, "rows": M, "out_features": N, "in_features": K, "weight_MB": N * K * 2 / 1e6}
        if args.small:  # one launch per shape with the library's own split, for a profiler
            ops.dense_gemm(x, w, out, status, workspace=gws)
            torch.cuda.synchronize()
            print(json.dumps({**row, "case": "dense --small", "launches": 1}))
            continue
        for ks in (0, 1, 2, 4, 8):
            if ks and (K // 64) % ks:
                continue
            med, _ = timer(lambda: ops.dense_gemm(x, w, out, status, k_split=ks, workspace=gws))
            row["us_auto" if ks == 0 else f"us_split{ks}"] = med
        lib, _ = timer(lambda: torch.matmul(x, w.t(), out=out))
        row.update({"us_library": lib, "GBs_auto": N * K * 2 / row["us_auto"] / 1e3, "peak_GBs": peak, "peak_source": src})
        print(json.dumps(row))
    x = torch.randn(M, H, generator=g, device=DEV).bfloat16()
    w = (torch.randn(args.vocab, H, generator=g, device=DEV) * 0.02).bfloat16()
    ws = ops.lm_head_argmax_workspace(DEV)
    tok = torch.empty(M, dtype=torch.int64, device=DEV)
    if args.small:
        ops.lm_head_argmax(x, w, ws, tok, status)
        torch.cuda.synchronize()
        ops.read_status(status, "dense")
        print(json.dumps({"case": "dense --small", "what": "lm_head + arg-max", "launches": 1}))
        return
    med, _ = timer(lambda: ops.lm_head_argmax(x, w, ws, tok, status))
    lib, _ = timer(lambda: torch.matmul(x, w.t()).argmax(dim=-1))
    ops.read_status(status, "dense")
    print(json.dumps({"case": "dense", "what": "lm_head + arg-max", "rows": M, "vocab": args.vocab, "hidden": H,
                      "weight_MB": args.vocab * H * 2 / 1e6, "us": med, "us_library_matmul_then_argmax": lib,
                      "GBs": args.vocab * H * 2 / med / 1e3, "frac_of_hbm_peak": args.vocab * H * 2 / med / 1e3 / peak,
                      "peak_GBs": peak, "peak_source": src}))


# ------------------------------------------------------------ dense FP8 peak --
def run_fp8peak(args) -> None:
    """What the library's dense e4m3 x e4m3 -> bf16 GEMM reaches on this GPU (per-tensor scales, no block
    scales): the practical tensor-core ceiling that the block-scaled MoE GEMM is compared with."""
    n = args.size
    g = torch.Generator(device=DEV).manual_seed(0)
    a = torch.randn(n, n, generator=g, device=DEV).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, generator=g, device=DEV).to(torch.float8_e4m3fn)
    one = torch.ones((), device=DEV)
    fn = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    med, mn = Timer(args.iters, flush=False)(fn, warm=5)
    x = torch.randn(n, n, generator=g, device=DEV).bfloat16()
    y = torch.randn(n, n, generator=g, device=DEV).bfloat16()
    med16, _ = Timer(args.iters, flush=False)(lambda: torch.matmul(x, y.t()), warm=5)
    print(json.dumps({"case": "fp8peak", "size": n, "fp8_us_median": med, "fp8_TFLOPs": 2 * n ** 3 / med / 1e6,
                      "fp8_TFLOPs_best": 2 * n ** 3 / mn / 1e6, "bf16_TFLOPs": 2 * n ** 3 / med16 / 1e6,
                      "note": "library GEMMs (cuBLASLt through torch), timed in isolation"}))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="case", required=True)
    a = sub.add_parser("attn")
    a.add_argument("--batch", type=int, default=64)
    a.add_argument("--q-heads", type=int, default=32)
    a.add_argument("--kv-heads", type=int, default=4)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--ctx-min", type=int, default=512)
    a.add_argument("--ctx-max", type=int, default=8192)
    a.add_argument("--share-group", type=int, default=8)
    a.add_argument("--share-tokens", type=int, default=1024)
    a.add_argument("--split-tokens", type=int, default=0)
    m = sub.add_parser("moe")
    m.add_argument("--tokens", default=MOE_TOKENS_DEFAULT, help="token counts; with --small only the first (default 64)")
    m.add_argument("--tiled", action="store_true", help="weights stored as contiguous 128x128 blocks")
    e = sub.add_parser("ep")
    e.add_argument("--world", type=int, default=8)
    e.add_argument("--tokens-per-rank", type=int, default=256)
    for p in (m, e):
        p.add_argument("--experts", type=int, default=128)
        p.add_argument("--top-k", type=int, default=8)
        p.add_argument("--hidden", type=int, default=2048)
        p.add_argument("--inter", type=int, default=768)
    pf = sub.add_parser("prefill")
    pf.add_argument("--chunk", type=int, default=1024)
    pf.add_argument("--first", default="0,1024,7168", help="tokens already in the sequence, comma separated")
    pf.add_argument("--q-heads", type=int, default=32)
    pf.add_argument("--kv-heads", type=int, default=4)
    pf.add_argument("--head-dim", type=int, default=128)
    pf.add_argument("--iters", type=int, default=10)
    pf.add_argument("--small", action="store_true", help="three launches (for a profiler)")
    d = sub.add_parser("dense")
    d.add_argument("--rows", type=int, default=256)
    d.add_argument("--hidden", type=int, default=2048)
    d.add_argument("--q-heads", type=int, default=32)
    d.add_argument("--kv-heads", type=int, default=4)
    d.add_argument("--head-dim", type=int, default=128)
    d.add_argument("--experts", type=int, default=128)
    d.add_argument("--vocab", type=int, default=151936)
    d.add_argument("--iters", type=int, default=20)
    d.add_argument("--small", action="store_true", help="one launch per shape (for a profiler)")
    f = sub.add_parser("fp8peak")
    f.add_argument("--size", type=int, default=8192)
    f.add_argument("--iters", type=int, default=20)
    f.add_argument("--small", action="store_true", help=argparse.SUPPRESS)
    for p in (a, m, e):
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--small", action="store_true", help="a few launches on a small case (for a profiler)")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("microbench.py needs a CUDA device")
    {"attn": run_attn, "moe": run_moe, "ep": run_ep, "fp8peak": run_fp8peak, "dense": run_dense, "prefill": run_prefill}[args.case](args)


if __name__ == "__main__":
    main()
