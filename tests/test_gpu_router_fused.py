"""Residual add + RMSNorm + router projection + top-k as one kernel through the C-ABI (B200), against the
separate kernels (b200_add_rmsnorm) and the CPU oracle of the router
(transformers Qwen3MoeTopKRouter, restated in oracle.route_ref)."""
import numpy as np
import pytest
import torch

from conftest import rel_err
import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def make(T, H, E, seed, with_delta=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).bfloat16()
    delta = (torch.randn(T, H, generator=g) * 0.5).bfloat16() if with_delta else None
    nw = (1.0 + 0.1 * torch.randn(H, generator=g)).bfloat16()
    rw = (torch.randn(E, H, generator=g) * 0.05).bfloat16()
    return x, delta, nw, rw


@pytest.mark.parametrize("T,H,E,K", [(256, 2048, 128, 8), (1, 2048, 128, 8), (37, 4096, 128, 8), (5, 512, 16, 4),
                                     (300, 2048, 128, 8), (16, 2048, 48, 6)])
@pytest.mark.parametrize("with_delta", [True, False])
def test_fused_norm_router_topk(ops, T, H, E, K, with_delta):
    assert ops.add_rmsnorm_route_supported(H, E, K)
    x, delta, nw, rw = make(T, H, E, seed=T + H + E, with_delta=with_delta)
    xd = x.to(DEV).clone()
    h, ids, w, logits = ops.add_rmsnorm_route(xd, None if delta is None else delta.to(DEV), nw.to(DEV), 1e-6, rw.to(DEV),
                                              K, True, want_logits=True)
    # the separate kernels on the same inputs
    x2 = x.to(DEV).clone()
    h_ref = ops.add_rmsnorm(x2, None if delta is None else delta.to(DEV), nw.to(DEV), 1e-6)
    assert torch.equal(xd, x2)                       # the residual stream is exact (bf16 add)
    same = (h == h_ref).float().mean()
    assert float(same) > 0.999 and rel_err(h, h_ref) < 4e-3   # the sum of squares is taken in another order: rare 1-ulp flips
    # logits: fp32 product of the kernel's own normed rows with the bf16 router matrix
    want = h.float().cpu() @ rw.float().t()
    assert rel_err(logits, want) < 1e-4
    # routing of exactly those logits, bit-exact in ids
    rid, rwt = oracle.route_ref(logits.cpu(), K, True)
    assert torch.equal(ids.cpu(), rid)
    np.testing.assert_allclose(w.cpu().numpy(), rwt.numpy(), rtol=3e-6, atol=1e-9)


def test_rows_beyond_num_valid_get_no_expert(ops):
    T, H, E, K, n_valid = 40, 2048, 128, 8, 23
    x, delta, nw, rw = make(T, H, E, seed=1)
    nv = torch.tensor([n_valid], dtype=torch.int32, device=DEV)
    h, ids, w = ops.add_rmsnorm_route(x.to(DEV), delta.to(DEV), nw.to(DEV), 1e-6, rw.to(DEV), K, True, num_valid=nv)
    h2, ids2, w2 = ops.add_rmsnorm_route(x.to(DEV), delta.to(DEV), nw.to(DEV), 1e-6, rw.to(DEV), K, True)
    assert torch.equal(ids[:n_valid], ids2[:n_valid]) and torch.equal(w[:n_valid], w2[:n_valid])
    assert bool((ids[n_valid:] == -1).all()) and bool((w[n_valid:] == 0).all())
    assert torch.equal(h, h2)  # the norm itself is not masked: the rows are padding, their values unused


def test_repeatable_and_independent_of_the_batch_around_a_row(ops):
    """A row's result does not depend on which other rows share its cluster (graphs of different batch sizes
    must agree bit for bit)."""
    T, H, E, K = 50, 2048, 128, 8
    x, delta, nw, rw = make(T, H, E, seed=2)
    a = ops.add_rmsnorm_route(x.to(DEV), delta.to(DEV), nw.to(DEV), 1e-6, rw.to(DEV), K, True, want_logits=True)
    b = ops.add_rmsnorm_route(x[:19].contiguous().to(DEV), delta[:19].contiguous().to(DEV), nw.to(DEV), 1e-6, rw.to(DEV),
                              K, True, want_logits=True)
    for u, v in zip(a, b):
        assert torch.equal(u[:19], v)


def test_unsupported_shapes_are_refused(ops):
    assert not ops.add_rmsnorm_route_supported(768, 128, 8)     # hidden not a multiple of 512
    assert not ops.add_rmsnorm_route_supported(2048, 256, 8)    # more than 128 experts
    x, delta, nw, rw = make(4, 768, 16, seed=3)
    with pytest.raises(Exception, match="multiple of 512"):
        ops.add_rmsnorm_route(x.to(DEV), None, nw.to(DEV), 1e-6, rw.to(DEV), 4)
