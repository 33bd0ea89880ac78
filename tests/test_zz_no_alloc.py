"""The allocation-free attention entry point against the regular one (B200).

b200_paged_attn_decode_static is for callers that hold no device allocator when
they need attention (a fully pre-partitioned memory pool, a plugin that is only
lent its input/output buffers, code inside a stream capture): its split partials
live in a fixed array inside the library.  The file sorts last on purpose, so a
run that stops at the first failure has already run every other test.  It must
pass alone in a fresh process and after the rest of the suite.
"""
import ctypes

import pytest
import torch

from conftest import pkg, rel_err
import oracle
from test_gpu_attention import build_case

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call_static(lib, q, kp, vp, table, ctx, out, status, scale, split):
    B, Hq, D = q.shape
    nb, Hkv, page, _ = kp.shape
    return lib.b200_paged_attn_decode_static(
        q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), ctx.data_ptr(), out.data_ptr(),
        status.data_ptr(), B, Hq, Hkv, D, page, nb, table.shape[1], ctypes.c_float(scale), split,
        torch.cuda.current_stream().cuda_stream)


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row(ops):
    lib = pkg("_lib").load()
    lens1 = [1, 17, 300, 1029, 64, 640, 2048, 77]
    lens2 = [900, 5, 128, 33, 1500, 16, 257, 1024]  # a second call re-uses the same scratch with other contents
    for lens, seed, split in ((lens1, 21, 256), (lens2, 22, 128)):
        q, kp, vp, table, ctx = [t.to(DEV) for t in build_case(len(lens), 32, 4, 128, lens, seed=seed)]
        scale = 128 ** -0.5
        ws = ops.paged_attn_workspace(len(lens), 32, 128, table.shape[1], 16, split, DEV)
        ref = ops.paged_attn_decode(q, kp, vp, table, ctx, scale, split, ws)
        ops.read_status(ws, "workspace entry")
        out = torch.full_like(q, float("nan"))
        status = torch.zeros(64, dtype=torch.int32, device=DEV)
        rc = _call_static(lib, q, kp, vp, table, ctx, out, status, scale, split)
        assert rc == 0, lib.b200_last_error_detail()
        ops.read_status(status, "static entry")
        # same kernels on the same inputs: well inside the 1e-2 bound the attention tests use
        err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        assert err < 1e-2
        assert torch.equal(out, ref)


def test_static_scratch_entry_against_the_oracle_on_a_large_batch_without_a_status_word(ops):
    """128 rows: above the batch size at which the workspace entry point switches to another pipeline shape
    (three shallow CTAs per SM up to 96 rows, two deeper ones above; this entry point always takes the second),
    so here the comparison is with the CPU oracle as well, and the status word is left out (NULL is allowed:
    findings are then not recorded)."""
    lib = pkg("_lib").load()
    rng = torch.Generator().manual_seed(5)
    lens = torch.randint(1, 700, (128,), generator=rng).tolist()
    q, kp, vp, table, ctx = build_case(128, 32, 4, 128, lens, seed=23)
    ref = oracle.paged_attn_ref(q, kp, vp, table, ctx, 128 ** -0.5)
    q, kp, vp, table, ctx = [t.to(DEV) for t in (q, kp, vp, table, ctx)]
    out = torch.full_like(q, float("nan"))
    B, Hq, D = q.shape
    rc = lib.b200_paged_attn_decode_static(
        q.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), ctx.data_ptr(), out.data_ptr(), None,
        B, Hq, 4, D, 16, kp.shape[0], table.shape[1], ctypes.c_float(128 ** -0.5), 128,
        torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.b200_last_error_detail()
    torch.cuda.synchronize()
    assert rel_err(out, ref) < 1e-2
    ws = ops.paged_attn_workspace(B, Hq, D, table.shape[1], 16, 128, DEV)
    same = ops.paged_attn_decode(q, kp, vp, table, ctx, 128 ** -0.5, 128, ws)
    assert torch.equal(out, same)  # 128 rows take the same pipeline shape in both entry points

    # a small batch goes through different pipeline shapes in the two entry points: equal within the bound
    lens = [900, 5, 128, 33, 1500, 16, 257, 1024]
    q, kp, vp, table, ctx = build_case(8, 32, 4, 128, lens, seed=24)
    ref = oracle.paged_attn_ref(q, kp, vp, table, ctx, 128 ** -0.5)
    q, kp, vp, table, ctx = [t.to(DEV) for t in (q, kp, vp, table, ctx)]
    out = torch.full_like(q, float("nan"))
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    assert _call_static(lib, q, kp, vp, table, ctx, out, status, 128 ** -0.5, 256) == 0
    ops.read_status(status, "static entry")
    assert rel_err(out, ref) < 1e-2


def test_static_scratch_entry_refuses_what_does_not_fit(ops):
    lib = pkg("_lib").load()
    lens = [64] * 64
    q, kp, vp, table, ctx = [t.to(DEV) for t in build_case(64, 32, 4, 128, lens, seed=1)]
    wide = torch.zeros(64, 4096, dtype=torch.int32, device=DEV)  # a 65536-token table at 16-token splits: > 32 MiB of partials
    wide[:, : table.shape[1]] = table
    out = torch.empty_like(q)
    status = torch.zeros(64, dtype=torch.int32, device=DEV)
    rc = _call_static(lib, q, kp, vp, wide, ctx, out, status, 0.1, 16)
    assert rc == -3 and b"built-in scratch" in lib.b200_last_error_detail()
    f32 = q.float()
    rc = lib.b200_paged_attn_decode_static(
        f32.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(), ctx.data_ptr(), out.data_ptr(), None,
        64, 32, 4, 96, 16, kp.shape[0], table.shape[1], ctypes.c_float(0.1), 64, None)
    assert rc == -1 and b"split-K kernel" in lib.b200_last_error_detail()
