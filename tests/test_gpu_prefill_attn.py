"""Tiled causal prompt attention over KV pages through the C-ABI (B200) vs the CPU oracle, which is pinned on
transformers eager attention with the causal mask over the reference's own page gather
(tests/golden/attn_prefill_d64.npz, tests/test_oracle_golden.py)."""
import numpy as np
import pytest
import torch

from conftest import golden, rel_err
import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-2  # max |err| / max |ref| for bf16 outputs


def test_golden_suffix_on_a_cached_prefix(ops):
    g = golden("attn_prefill_d64.npz")
    q, kp, vp = (torch.from_numpy(g[k]).bfloat16() for k in ("q", "k_pool", "v_pool"))
    row = torch.from_numpy(g["table_row"])
    first, scale = int(g["first_pos"]), float(g["scale"])
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    out = ops.paged_attn_prefill(q.to(DEV), kp.to(DEV), vp.to(DEV), row.to(DEV), first, scale, status)
    ops.read_status(status, "paged_attn_prefill")
    ref = oracle.paged_prefill_ref(q, kp, vp, row.tolist(), first, scale)  # same bf16 inputs
    assert rel_err(out, ref) < TOL
    assert rel_err(out, torch.from_numpy(g["out"])) < 2e-2  # and close to the fp32 run of the reference's path


def case(hq, hkv, d, first, rows, seed):
    g = torch.Generator().manual_seed(seed)
    total = first + rows
    n_pages = (total + 15) // 16
    ids = torch.randperm(n_pages + 7, generator=g)[:n_pages].to(torch.int32)
    kp = torch.randn(n_pages + 7, hkv, 16, d, generator=g).bfloat16()
    vp = torch.randn(n_pages + 7, hkv, 16, d, generator=g).bfloat16()
    q = torch.randn(rows, hq, d, generator=g).bfloat16()
    row = torch.zeros(n_pages + 3, dtype=torch.int32)
    row[:n_pages] = ids
    return q, kp, vp, row


@pytest.mark.parametrize("hq,hkv,d", [(32, 4, 128), (64, 4, 128), (8, 2, 64)])
@pytest.mark.parametrize("first,rows", [(0, 1), (0, 17), (100, 128), (37, 300), (1000, 16), (2047, 33)])
def test_chunk_shapes_and_positions(ops, hq, hkv, d, first, rows):
    q, kp, vp, row = case(hq, hkv, d, first, rows, seed=first + rows)
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    out = ops.paged_attn_prefill(q.to(DEV), kp.to(DEV), vp.to(DEV), row.to(DEV), first, d ** -0.5, status)
    ops.read_status(status, "paged_attn_prefill")
    ref = oracle.paged_prefill_ref(q, kp, vp, row.tolist(), first, d ** -0.5)
    assert rel_err(out, ref) < TOL
    # row by row too: a wrong causal edge shows in single rows long before it moves the tensor-wide maximum
    per_row = (out.float().cpu() - ref).abs().amax(dim=(1, 2)) / ref.abs().amax()
    assert float(per_row.max()) < TOL


def test_same_rows_as_the_decode_kernel_gives_them_one_by_one(ops):
    """The row of position p is decode attention at context length p + 1."""
    hq, hkv, d, first, rows = 32, 4, 128, 200, 64
    q, kp, vp, row = case(hq, hkv, d, first, rows, seed=5)
    qd, kd, vd, rd = q.to(DEV), kp.to(DEV), vp.to(DEV), row.to(DEV)
    out = ops.paged_attn_prefill(qd, kd, vd, rd, first, d ** -0.5)
    table = rd.view(1, -1).expand(rows, -1).contiguous()
    lens = torch.arange(first + 1, first + rows + 1, dtype=torch.int32, device=DEV)
    dec = ops.paged_attn_decode(qd, kd, vd, table, lens, d ** -0.5)
    assert rel_err(out, dec) < 5e-3


def test_positions_past_the_table_and_bad_pages_are_reported_not_read(ops):
    q, kp, vp, row = case(32, 4, 128, 0, 40, seed=7)
    with pytest.raises(Exception, match="do not fit"):
        ops.paged_attn_prefill(q.to(DEV), kp.to(DEV), vp.to(DEV), row.to(DEV), row.numel() * 16 - 10, 0.1)
    bad = row.clone()
    bad[1] = 10_000
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    ops.paged_attn_prefill(q.to(DEV), kp.to(DEV), vp.to(DEV), bad.to(DEV), 0, 0.1, status)
    with pytest.raises(Exception, match="block table entry"):
        ops.read_status(status, "paged_attn_prefill")
