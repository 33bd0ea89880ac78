"""Paged decode attention and KV append through the C-ABI vs the CPU oracle (B200)."""
import numpy as np
import pytest
import torch

from conftest import golden, rel_err
import oracle

pytestmark = pytest.mark.gpu
TOL_BF16 = 1e-2  # max |err| / max |ref|, the bound the spec gives for bf16 outputs


def build_case(B, Hq, Hkv, D, ctx_lens, seed, group_share=0, shared_tokens=0, page=16, dtype=torch.bfloat16,
               const_v=None):
    """Seeded pools + shuffled block tables; rows of a share group reuse their first full pages."""
    g = torch.Generator().manual_seed(seed)
    rng = np.random.default_rng(seed)
    n_pages = [(L + page - 1) // page for L in ctx_lens]
    max_pages = max(1, max(n_pages))
    total = sum(n_pages) + 8
    perm = rng.permutation(total).tolist()
    table = np.zeros((B, max_pages), dtype=np.int32)
    shared = {}
    for b, L in enumerate(ctx_lens):
        grp = b // group_share if group_share else -1
        for p in range(n_pages[b]):
            full = (p + 1) * page <= L
            if group_share and full and (p + 1) * page <= shared_tokens:
                key = (grp, p)
                if key not in shared:
                    shared[key] = perm.pop()
                table[b, p] = shared[key]
            else:
                table[b, p] = perm.pop()
    k_pool = torch.randn(total, Hkv, page, D, generator=g).to(dtype)
    v_pool = torch.randn(total, Hkv, page, D, generator=g).to(dtype)
    if const_v is not None:
        v_pool[:] = const_v.to(dtype).view(1, 1, 1, D)
    q = torch.randn(B, Hq, D, generator=g).to(dtype)
    return q, k_pool, v_pool, torch.from_numpy(table), torch.tensor(ctx_lens, dtype=torch.int32)


def run(ops, q, k_pool, v_pool, table, lens, split_tokens=None):
    dev = "cuda"
    D, page = q.shape[-1], k_pool.shape[2]
    B, Hq = q.shape[:2]
    st = split_tokens or ops.default_split_tokens(B, k_pool.shape[1], table.shape[1] * page)
    ws = ops.paged_attn_workspace(B, Hq, D, table.shape[1], page, st, dev)
    out = ops.paged_attn_decode(q.to(dev), k_pool.to(dev), v_pool.to(dev), table.to(dev), lens.to(dev),
                                D ** -0.5, split_tokens=st, workspace=ws)
    ops.read_status(ws, "paged_attn_decode")
    return out


@pytest.mark.parametrize("name", ["attn_d64.npz", "attn_d128.npz"])
def test_golden_fp32_generic_kernel(ops, name):
    g = golden(name)
    t = lambda k: torch.from_numpy(g[k])
    out = run(ops, t("q"), t("k_pool"), t("v_pool"), t("block_table"), t("ctx_lens"))
    np.testing.assert_allclose(out.cpu().numpy(), g["out"], rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("name", ["attn_d64.npz", "attn_d128.npz"])
@pytest.mark.parametrize("split", [64, 128])
def test_golden_bf16_tma_kernel(ops, name, split):
    g = golden(name)
    t = lambda k: torch.from_numpy(g[k])
    q, kp, vp = t("q").bfloat16(), t("k_pool").bfloat16(), t("v_pool").bfloat16()
    out = run(ops, q, kp, vp, t("block_table"), t("ctx_lens"), split_tokens=split)
    ref = oracle.paged_attn_ref(q, kp, vp, t("block_table"), t("ctx_lens"), float(g["scale"]))
    assert rel_err(out, ref) < TOL_BF16
    # and still close to the reference's fp32 answer on unrounded inputs
    assert rel_err(out, torch.from_numpy(g["out"])) < 3e-2


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 4, 128), (8, 2, 64), (64, 4, 128), (4, 4, 128), (16, 4, 64),
                                       (8, 1, 128), (64, 8, 128), (16, 2, 128), (16, 1, 64), (32, 8, 64), (12, 4, 128)])
def test_ragged_lengths_and_split_boundaries(ops, Hq, Hkv, D):
    lens = [1, 15, 16, 17, 63, 64, 65, 255, 256, 257, 300, 511, 512, 513, 1000, 0]
    q, kp, vp, table, ctx = build_case(len(lens), Hq, Hkv, D, lens, seed=7)
    out = run(ops, q, kp, vp, table, ctx, split_tokens=256)
    ref = oracle.paged_attn_ref(q, kp, vp, table, ctx, D ** -0.5)
    assert rel_err(out, ref) < TOL_BF16
    assert float(out[-1].float().abs().max()) == 0.0  # empty row -> zeros


def test_radix_shared_prefix_pages(ops):
    rng = np.random.default_rng(0)
    lens = rng.integers(200, 1500, size=16).tolist()
    q, kp, vp, table, ctx = build_case(16, 32, 4, 128, lens, seed=3, group_share=8, shared_tokens=512)
    assert len(np.unique(table.numpy()[:8, :8])) < 64  # pages really are shared
    out = run(ops, q, kp, vp, table, ctx)
    ref = oracle.paged_attn_ref(q, kp, vp, table, ctx, 128 ** -0.5)
    assert rel_err(out, ref) < TOL_BF16


def test_page_placement_does_not_change_a_single_bit(ops):
    """Block-table gather is exact: moving pages around in the pool gives identical bits."""
    lens = [700, 33, 1024, 129]
    q, kp, vp, table, ctx = build_case(4, 32, 4, 128, lens, seed=11)
    out1 = run(ops, q, kp, vp, table, ctx, split_tokens=128)
    perm = torch.randperm(kp.shape[0], generator=torch.Generator().manual_seed(5))
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel())
    out2 = run(ops, q, kp[perm], vp[perm], inv[table.long()].to(torch.int32), ctx, split_tokens=128)
    assert torch.equal(out1, out2)


def test_full_size_config2_properties(ops):
    """BASELINE config 2 at full size (64 rows, 512..8192 tokens, groups of 8 share 1024 tokens):
    constant V rows must come back exactly (softmax weights sum to 1), and 8 sampled rows match the oracle."""
    rng = np.random.default_rng(0)
    lens = rng.integers(512, 8193, size=64).tolist()
    c = torch.linspace(-2, 2, 128)
    q, kp, vp, table, ctx = build_case(64, 32, 4, 128, lens, seed=0, group_share=8, shared_tokens=1024, const_v=c)
    out = run(ops, q, kp, vp, table, ctx)
    want = c.bfloat16().float().view(1, 1, 128).expand(64, 32, 128)
    assert float((out.float().cpu() - want).abs().max()) <= 2 ** -6  # one bf16 ulp at |2|
    g = torch.Generator().manual_seed(1)
    vp2 = torch.randn(vp.shape, generator=g).bfloat16()
    out2 = run(ops, q, kp, vp2, table, ctx)
    rows = [0, 7, 8, 21, 35, 42, 56, 63]
    ref = oracle.paged_attn_ref(q[rows], kp, vp2, table[rows], ctx[rows], 128 ** -0.5)
    assert rel_err(out2[rows], ref) < TOL_BF16


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_kv_append_writes_the_page_slot(ops, dtype):
    lens = [5, 16, 31, 100]
    q, kp, vp, table, ctx = build_case(4, 8, 2, 64, [l + 1 for l in lens], seed=9, dtype=dtype)
    dev = "cuda"
    kp_d, vp_d = kp.to(dev), vp.to(dev)
    g = torch.Generator().manual_seed(2)
    k_new = torch.randn(4, 2, 64, generator=g).to(dtype)
    v_new = torch.randn(4, 2, 64, generator=g).to(dtype)
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    ops.kv_append(k_new.to(dev), v_new.to(dev), kp_d, vp_d, table.to(dev), torch.tensor(lens, dtype=torch.int32, device=dev), status)
    ops.read_status(status, "kv_append")
    for b, pos in enumerate(lens):
        page_id = int(table[b, pos // 16])
        kp[page_id, :, pos % 16, :] = k_new[b]
        vp[page_id, :, pos % 16, :] = v_new[b]
    assert torch.equal(kp_d.cpu(), kp) and torch.equal(vp_d.cpu(), vp)
    out = ops.paged_attn_decode(q.to(dev), kp_d, vp_d, table.to(dev), ctx.to(dev), 0.125)
    ref = oracle.paged_attn_ref(q, kp, vp, table, ctx, 0.125)
    assert rel_err(out, ref) < (TOL_BF16 if dtype == torch.bfloat16 else 1e-5)


def test_bad_block_id_is_reported_not_faulted(ops):
    """An id outside the pool is clamped on the device and reported through the status word."""
    q, kp, vp, table, ctx = build_case(2, 32, 4, 128, [40, 40], seed=4)
    table[1, 1] = kp.shape[0] + 5
    dev = "cuda"
    ws = ops.paged_attn_workspace(2, 32, 128, table.shape[1], 16, 64, dev)
    ops.paged_attn_decode(q.to(dev), kp.to(dev), vp.to(dev), table.to(dev), ctx.to(dev), 0.1, split_tokens=64, workspace=ws)
    with pytest.raises(Exception, match="block table"):
        ops.read_status(ws)


def test_host_side_argument_errors(ops):
    q, kp, vp, table, ctx = build_case(2, 32, 4, 128, [40, 40], seed=4)
    dev = "cuda"
    with pytest.raises(Exception, match="split_tokens"):
        ops.paged_attn_decode(q.to(dev), kp.to(dev), vp.to(dev), table.to(dev), ctx.to(dev), 0.1, split_tokens=100)
    tiny = torch.zeros(8, dtype=torch.uint8, device=dev)
    with pytest.raises(Exception, match="workspace"):
        ops.paged_attn_decode(q.to(dev), kp.to(dev), vp.to(dev), table.to(dev), ctx.to(dev), 0.1, split_tokens=64, workspace=tiny)


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 4, 128), (8, 2, 64), (16, 4, 128)])
@pytest.mark.parametrize("split", [64, 256])
def test_pair_form_gives_the_same_bits_as_one_row_per_cta(ops, Hq, Hkv, D, split):
    """b200_paged_attn_decode_pairs: rows 2i and 2i+1 share table row 2i and are computed by one CTA (the second
    row in the upper half of the MMA tile).  Every row must come out bit-identical to the one-row kernel: a
    prompt's consecutive lengths, equal lengths, a second row that starts in a later split than the first
    ends, empty rows, and an odd row count."""
    lens_pairs = [(1, 2), (15, 16), (16, 17), (63, 64), (64, 65), (200, 201), (300, 300), (7, 500), (500, 7),
                  (0, 40), (40, 0), (0, 0), (129, 130), (511, 512)]
    lens = [l for pr in lens_pairs for l in pr] + [333]  # odd count: the last pair has one row
    B = len(lens)
    share = [max(lens[2 * (i // 2)], lens[min(B - 1, 2 * (i // 2) + 1)]) for i in range(B)]
    q, kp, vp, table, ctx = build_case(B, Hq, Hkv, D, share, seed=B + Hq)  # pages for the longer row of a pair
    for i in range(1, B, 2):
        table[i] = table[i - 1]  # the pair shares the first row's table
    ctx = torch.tensor(lens, dtype=torch.int32)
    dev = "cuda"
    q, kp, vp, table, ctx = [t.to(dev) for t in (q, kp, vp, table, ctx)]
    ws = ops.paged_attn_workspace(B, Hq, D, table.shape[1], 16, split, dev)
    one = ops.paged_attn_decode(q, kp, vp, table, ctx, D ** -0.5, split, ws).clone()
    ops.read_status(ws, "one row per CTA")
    ws2 = ops.paged_attn_workspace(B, Hq, D, table.shape[1], 16, split, dev)
    scrambled = table.clone()
    scrambled[1::2] = 0  # odd table rows are not read by the pair form
    two = ops.paged_attn_decode(q, kp, vp, scrambled, ctx, D ** -0.5, split, ws2, pairs=True)
    ops.read_status(ws2, "pairs")
    assert torch.equal(one, two), f"rows differ: {(one != two).flatten(1).any(1).nonzero().flatten().tolist()}"
    assert ops.paged_attn_pairs_supported(Hq, Hkv, D, 16, torch.bfloat16)
    assert not ops.paged_attn_pairs_supported(64, 4, 128, 16, torch.bfloat16)  # 16 heads per kv head: no idle rows
