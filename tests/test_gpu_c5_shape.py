"""One layer at the Qwen3-235B-A22B shape (BASELINE config 5) through the C-ABI vs the CPU oracle (B200):
64 query / 4 kv heads of 128 for attention, hidden 4096 with expert intermediate 1536 for the FP8 MoE layer.
The model itself needs several GPUs; its layer kernels are checked here at their real widths on one."""
import numpy as np
import pytest
import torch

from conftest import rel_err
import oracle
from test_gpu_attention import build_case, run

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-2  # max |err| / max |ref| for bf16 outputs


def test_attention_with_sixteen_query_heads_per_kv_head(ops):
    lens = [1, 16, 17, 700, 2049, 4096, 33, 1500]
    q, kp, vp, table, ctx = build_case(len(lens), 64, 4, 128, lens, seed=51, group_share=4, shared_tokens=512)
    ref = oracle.paged_attn_ref(q, kp, vp, table, ctx, 128 ** -0.5)
    for split in (None, 256, 4096):  # library default, many splits, no split
        out = run(ops, q, kp, vp, table, ctx, split_tokens=split)
        assert rel_err(out, ref) < TOL, f"split_tokens {split}"


@pytest.mark.parametrize("T", [1, 48, 300])
def test_fp8_moe_layer_at_hidden_4096_intermediate_1536(ops, T):
    E, K, H, I = 16, 8, 4096, 1536  # the real expert size; 16 of the model's 128 experts keep the oracle quick
    g = torch.Generator().manual_seed(52)
    w13q, w13s = oracle.quantize_weight_ref(torch.randn(E, 2 * I, H, generator=g) * 0.02)
    w2q, w2s = oracle.quantize_weight_ref(torch.randn(E, H, I, generator=g) * 0.02)
    x = torch.randn(T, H, generator=g).bfloat16()
    logits = torch.randn(T, E, generator=g)
    ws = ops.moe_fp8_workspace(T, E, K, H, I, DEV)
    y = ops.moe_fp8_forward(x.to(DEV), logits.to(DEV), w13q.to(DEV), w13s.to(DEV), w2q.to(DEV), w2s.to(DEV), K, True, ws)
    ops.read_status(ws, "FP8 MoE layer")
    ref, parts = oracle.moe_fp8_ref(x, logits, w13q, w13s, w2q, w2s, K, True, return_parts=True)
    assert rel_err(y, ref) < TOL
    # the integer side of the layer is exact at this shape too: ids, permutation, quantised activations
    ids, _ = ops.moe_route(logits.to(DEV), K, True)
    assert torch.equal(ids.cpu(), parts["ids"])
    p, xq, xs = ops.moe_permute_quant(ids, x.to(DEV), E)
    np.testing.assert_array_equal(p.row_of_pair.cpu().numpy(), parts["perm"]["row_of_pair"])
    tok = torch.from_numpy(parts["perm"]["sorted_pair_ids"]).long() // K
    np.testing.assert_array_equal(xq.cpu().numpy(), parts["xq"].view(torch.uint8)[tok].numpy())
    np.testing.assert_array_equal(xs.cpu().numpy(), parts["xs"][tok].numpy())
