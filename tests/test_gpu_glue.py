"""Fused residual+RMSNorm and q/k norm + RoPE + page write through the C-ABI vs the CPU oracle (B200)."""
import pytest
import torch

from conftest import rel_err
from oracle import glue_ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("rows,H", [(1, 2048), (256, 2048), (7, 512), (33, 4096)])
def test_add_rmsnorm(ops, rows, H):
    g = torch.Generator().manual_seed(rows + H)
    x = torch.randn(rows, H, generator=g).bfloat16()
    d = torch.randn(rows, H, generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    xd = x.to(DEV)
    out = ops.add_rmsnorm(xd, d.to(DEV), w.to(DEV), 1e-6)
    res = x + d  # bf16 add, as the model does
    assert torch.equal(xd.cpu(), res)  # residual stream updated in place, bit-exact
    ref = glue_ref.rms_norm_ref(res, w, 1e-6)
    assert rel_err(out, ref) < 1e-2
    assert (out.cpu() != ref).float().mean() < 0.02  # at most a last-bit difference on a few elements
    out2 = ops.add_rmsnorm(xd, None, w.to(DEV), 1e-6)  # no delta: x untouched
    assert torch.equal(xd.cpu(), res) and torch.equal(out2, out)


@pytest.mark.parametrize("B,Hq,Hkv,D", [(5, 32, 4, 128), (4, 8, 2, 64), (64, 64, 4, 128)])
def test_qk_norm_rope_append(ops, B, Hq, Hkv, D):
    g = torch.Generator().manual_seed(B + D)
    qkv = torch.randn(B, Hq + 2 * Hkv, D, generator=g).bfloat16()
    qw = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16()
    kw = (1 + 0.1 * torch.randn(D, generator=g)).bfloat16()
    max_pages = 8
    cos, sin = glue_ref.rope_tables_ref(D, 1e6, max_pages * 16)
    pos = torch.randint(0, max_pages * 16, (B,), generator=g).to(torch.int32)
    table = torch.randperm(B * max_pages, generator=g).view(B, max_pages).to(torch.int32)
    kp = torch.randn(B * max_pages, Hkv, 16, D, generator=g).bfloat16()
    vp = torch.randn(B * max_pages, Hkv, 16, D, generator=g).bfloat16()
    kd, vd = kp.to(DEV), vp.to(DEV)
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    q = ops.qk_norm_rope_append(qkv.to(DEV), qw.to(DEV), kw.to(DEV), cos.to(DEV), sin.to(DEV), pos.to(DEV),
                                table.to(DEV), kd, vd, Hq, 1e-6, status)
    ops.read_status(status, "qk_norm_rope_append")
    qr, kr, vr = glue_ref.qk_norm_rope_append_ref(qkv, qw, kw, cos, sin, pos, table, kp, vp, Hq, 1e-6)
    assert rel_err(q, qr) < 1e-2
    assert rel_err(kd, kr) < 1e-2
    assert torch.equal(vd.cpu(), vr)  # v is a plain copy into the slot: bit-exact
    untouched = torch.ones(B * max_pages, dtype=torch.bool)
    for b in range(B):
        untouched[int(table[b, int(pos[b]) // 16])] = False
    assert torch.equal(kd.cpu()[untouched], kp[untouched])  # no other page was written
