"""Dense bf16 projections and the fused lm_head arg-max through the C-ABI (B200) against an fp32 matmul of the
same bf16 inputs on the CPU - what the reference's model forward computes in its linear layers
(transformers Qwen3-MoE q/k/v/o projections, router gate, lm_head; torch_backend.py:314-321)."""
import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-2  # max |err| / max |ref| for bf16 outputs


def make(M, N, K, seed, wstd=0.02):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * wstd).bfloat16()
    return x, w, x.float() @ w.float().t()


@pytest.mark.parametrize("M,N,K", [
    (256, 5120, 2048),   # config 4: fused q/k/v projection at the full decode batch (K split over a cluster)
    (256, 2048, 4096),   # config 4: o projection
    (256, 128, 2048),    # config 4: router gate (one weight tile)
    (32, 9216, 4096),    # config 5: q/k/v projection, 32 rows per GPU
    (1, 5120, 2048),     # a single row
    (7, 768, 512),       # tiny model q/k/v
    (33, 200, 512),      # out_features not a multiple of the 128-row weight tile
    (300, 1024, 512),    # more rows than one MMA takes: two row tiles
    (1024, 1536, 1024),  # a prompt chunk: four row tiles, no K split
    (5, 4096, 512),      # tiny model lm_head as plain logits
])
def test_dense_gemm_matches_fp32_matmul(ops, M, N, K):
    x, w, ref = make(M, N, K, seed=M + N)
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    y = ops.dense_gemm(x.to(DEV), w.to(DEV), status=status)
    ops.read_status(status, "dense_gemm")
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert rel_err(y, ref) < TOL
    # bf16 rounding of an exact-enough fp32 sum: most elements are the correctly rounded value
    exact = (y.cpu() == ref.bfloat16()).float().mean()
    assert exact > 0.95


@pytest.mark.parametrize("k_split", [1, 2, 4, 8])
def test_every_k_split_gives_the_same_product_and_is_repeatable(ops, k_split):
    x, w, ref = make(64, 640, 2048, seed=3)
    xd, wd = x.to(DEV), w.to(DEV)
    a = ops.dense_gemm(xd, wd, k_split=k_split)
    b = ops.dense_gemm(xd, wd, k_split=k_split)
    assert torch.equal(a, b)  # the cluster fold sums the partials in rank order: no run-to-run difference
    assert rel_err(a, ref) < TOL


def test_dense_gemm_rejects_what_it_cannot_run(ops):
    x = torch.zeros(4, 96, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 96, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception, match="multiple of 64"):
        ops.dense_gemm(x, w)
    x = torch.zeros(4, 128, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception, match="k_split"):
        ops.dense_gemm(x, w, k_split=4)  # two K blocks cannot be split four ways


@pytest.mark.parametrize("M,V,K", [(256, 151936, 2048), (32, 151936, 4096), (5, 4096, 512), (3, 1000, 512), (1, 151936, 2048)])
def test_lm_head_argmax_picks_the_largest_logit(ops, M, V, K):
    x, w, ref = make(M, V, K, seed=V + M)
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    tok = ops.lm_head_argmax(x.to(DEV), w.to(DEV), status=status)
    ops.read_status(status, "lm_head_argmax")
    assert tok.dtype == torch.int64 and tok.shape == (M,)
    tok = tok.cpu()
    assert int(tok.min()) >= 0 and int(tok.max()) < V
    best = ref.max(dim=1).values
    chosen = ref[torch.arange(M), tok]
    # the kernel compares its own fp32 sums; an fp32 sum in another order may rank two near-equal logits the
    # other way, so the chosen logit must be the largest up to that rounding
    assert float((best - chosen).max()) <= 1e-4 * float(ref.abs().max())
    top2 = torch.topk(ref, 2, dim=1).values
    clear = (top2[:, 0] - top2[:, 1]) > 1e-3 * float(ref.abs().max())
    assert torch.equal(tok[clear], ref.argmax(dim=1)[clear])


def test_lm_head_argmax_ties_go_to_the_lower_token_id(ops):
    V, K = 3000, 128
    w = torch.zeros(V, K)
    x = torch.zeros(4, K)
    x[:, 0] = 1.0
    w[[17, 900, 2999], 0] = 2.0   # three equal maxima, in different weight tiles and CTAs
    w[5, 0] = 1.0
    x[1, 0] = -1.0                 # row 1: the maxima become minima; the largest is 0, first at token 0
    tok = ops.lm_head_argmax(x.bfloat16().to(DEV), w.bfloat16().to(DEV)).cpu().tolist()
    assert tok == [17, 0, 17, 17]


def test_lm_head_argmax_agrees_with_argmax_of_the_written_logits(ops):
    x, w, _ = make(64, 8192, 1024, seed=11)
    xd, wd = x.to(DEV), w.to(DEV)
    logits = ops.dense_gemm(xd, wd).float()
    tok = ops.lm_head_argmax(xd, wd)
    picked = logits[torch.arange(64, device=DEV), tok]
    # the written logits are rounded to bf16, which creates ties that the fp32 comparison does not see
    assert bool((picked == logits.max(dim=1).values).all())


@pytest.mark.parametrize("R,hq,hkv,K", [(256, 32, 4, 2048), (1, 32, 4, 2048), (37, 64, 4, 4096), (300, 8, 2, 512)])
def test_qkv_projection_with_norm_rope_and_page_write_equals_the_two_kernels(ops, R, hq, hkv, K):
    """b200_qkv_rope_append_gemm against b200_dense_gemm_bf16 (no K split) + b200_qk_norm_rope_append: the query
    rows and every page of both pools must come out bit for bit the same."""
    D, page, max_pages = 128, 16, 6
    assert ops.qkv_rope_append_supported(D, K)
    g = torch.Generator().manual_seed(R + K)
    x = torch.randn(R, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn((hq + 2 * hkv) * D, K, generator=g) * 0.03).bfloat16().to(DEV)
    qn = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16().to(DEV)
    kn = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16().to(DEV)
    ang = torch.arange(max_pages * page, dtype=torch.float32)[:, None] / (1e6 ** (torch.arange(0, D, 2) / D))[None, :]
    emb = torch.cat([ang, ang], dim=-1)
    cos, sin = emb.cos().bfloat16().to(DEV), emb.sin().bfloat16().to(DEV)
    pos = torch.randint(0, max_pages * page, (R,), generator=g).to(torch.int32).to(DEV)
    nb = R * max_pages + 3
    table = torch.randperm(nb, generator=g)[: R * max_pages].view(R, max_pages).to(torch.int32).to(DEV)
    pools = [torch.randn(nb, hkv, page, D, generator=g).bfloat16().to(DEV) for _ in range(2)]
    k1, v1, k2, v2 = pools[0].clone(), pools[1].clone(), pools[0].clone(), pools[1].clone()
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    q1 = ops.qkv_rope_append_gemm(x, w, qn, kn, cos, sin, pos, table, k1, v1, hq, 1e-6, status)
    ops.read_status(status, "qkv_rope_append_gemm")
    qkv = ops.dense_gemm(x, w, k_split=1).view(R, hq + 2 * hkv, D)
    q2 = ops.qk_norm_rope_append(qkv, qn, kn, cos, sin, pos, table, k2, v2, hq, 1e-6, status)
    ops.read_status(status, "qk_norm_rope_append")
    assert torch.equal(q1, q2)
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert not torch.equal(k1, pools[0])  # something was written


def test_qkv_projection_epilogue_reports_bad_positions_and_pages(ops):
    R, hq, hkv, K, D = 4, 32, 4, 2048, 128
    g = torch.Generator().manual_seed(0)
    x = torch.randn(R, K, generator=g).bfloat16().to(DEV)
    w = (torch.randn((hq + 2 * hkv) * D, K, generator=g) * 0.03).bfloat16().to(DEV)
    one = torch.ones(D, dtype=torch.bfloat16, device=DEV)
    cs = torch.ones(64, D, dtype=torch.bfloat16, device=DEV)
    pool = torch.zeros(8, hkv, 16, D, dtype=torch.bfloat16, device=DEV)
    table = torch.zeros(R, 4, dtype=torch.int32, device=DEV)
    table[2, 0] = 99  # outside the pool
    pos = torch.tensor([0, 1, 2, 3], dtype=torch.int32, device=DEV)
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    ops.qkv_rope_append_gemm(x, w, one, one, cs, cs, pos, table, pool, pool.clone(), hq, 1e-6, status)
    with pytest.raises(Exception, match="block table entry"):
        ops.read_status(status, "qkv_rope_append_gemm")
