"""The oracle against the golden vectors made from the real reference (CPU)."""
import numpy as np
import pytest
import torch

from conftest import golden
import oracle


def _attn(name, tol):
    g = golden(name)
    out = oracle.paged_attn_ref(
        torch.from_numpy(g["q"]), torch.from_numpy(g["k_pool"]), torch.from_numpy(g["v_pool"]),
        torch.from_numpy(g["block_table"]), torch.from_numpy(g["ctx_lens"]), float(g["scale"]))
    np.testing.assert_allclose(out.numpy(), g["out"], rtol=tol, atol=tol)


def test_paged_attention_d64_matches_reference_gather_and_eager_attention():
    _attn("attn_d64.npz", 2e-6)


def test_paged_attention_d128_matches_reference_gather_and_eager_attention():
    _attn("attn_d128.npz", 2e-6)


def test_gather_pages_partial_last_page():
    pool = torch.arange(3 * 2 * 4 * 2, dtype=torch.float32).reshape(3, 2, 4, 2)
    dense = oracle.gather_pages(pool, [2, 0], 6)
    assert dense.shape == (2, 6, 2)
    assert torch.equal(dense[:, :4], pool[2]) and torch.equal(dense[:, 4:], pool[0, :, :2])
    assert oracle.gather_pages(pool, [1], 0).shape == (2, 0, 2)


def _route(name):
    g = golden(name)
    logits = torch.from_numpy(g["logits"])
    K = g["topk_ids"].shape[1]
    ids, w = oracle.route_ref(logits, K, True)
    # torch.topk (what the reference's model uses) and the fixed tie rule agree on tie-free rows
    probs = torch.softmax(logits, -1)
    top = torch.topk(probs, K + 1, dim=-1).values
    tie_free = (top[:, :-1] != top[:, 1:]).all(dim=1).numpy()
    assert tie_free.mean() > 0.99
    np.testing.assert_array_equal(ids.numpy()[tie_free], g["topk_ids"][tie_free])
    np.testing.assert_allclose(w.numpy()[tie_free], g["topk_weights"][tie_free], rtol=1e-6, atol=1e-8)


def test_route_e128_k8_matches_hf_router():
    _route("route_e128k8.npz")


def test_route_e16_k4_matches_hf_router():
    _route("route_e16k4.npz")


def test_route_tie_rule_lower_expert_id_first():
    logits = torch.tensor([[0.0, 1.0, 1.0, -1.0, 1.0, 0.5, 1.0, 1.0]])
    ids, w = oracle.route_ref(logits, 3, True)
    assert ids.tolist() == [[1, 2, 4]]
    np.testing.assert_allclose(w.numpy(), np.full((1, 3), 1 / 3), rtol=1e-6)


def test_permute_is_stable_sort_by_expert():
    ids = torch.tensor([[3, 1], [1, 0], [3, 0], [1, 3]], dtype=torch.int32)
    p = oracle.permute_ref(ids, 4)
    assert p["expert_offsets"].tolist() == [0, 2, 5, 5, 8]
    assert p["sorted_pair_ids"].tolist() == [3, 5, 1, 2, 6, 0, 4, 7]
    assert p["row_of_pair"][p["sorted_pair_ids"]].tolist() == list(range(8))
    assert p["tiles"].tolist() == [[0, 0, 2, 0], [1, 2, 3, 0], [3, 5, 3, 0]]


def test_dense_experts_match_hf_eager_experts():
    g = golden("experts_dense.npz")
    out = oracle.moe_dense_ref(torch.from_numpy(g["x"]), torch.from_numpy(g["logits"]),
                               torch.from_numpy(g["gate_up_proj"]), torch.from_numpy(g["down_proj"]),
                               int(g["top_k"]))
    np.testing.assert_allclose(out.numpy(), g["out"], rtol=2e-5, atol=2e-6)


def test_weight_quant_matches_hf_fp8quantize_bit_exact():
    g = golden("fp8_weight_quant.npz")
    q, s = oracle.quantize_weight_ref(torch.from_numpy(g["w"]))
    np.testing.assert_array_equal(q.view(torch.uint8).numpy(), g["q"])
    np.testing.assert_array_equal(s.numpy(), g["scale_inv"])
    assert float(s[1, 0, 0]) == 1.0  # all-zero tile


def test_act_quant_round_trip_and_zero_group():
    torch.manual_seed(0)
    x = torch.randn(5, 256).to(torch.bfloat16)
    x[2, :128] = 0
    q, s = oracle.act_quant_ref(x)
    assert float(s[2, 0]) == 1.0 and int(q.view(torch.uint8)[2, :128].max()) == 0
    back = oracle.dequant_act(q, s)
    assert float((back - x.float()).abs().max() / x.float().abs().max()) < 0.07
    # the largest element of every group maps to +-448 exactly
    g = q.float().reshape(5, 2, 128).abs().amax(-1)
    assert torch.all((g == 448) | (g == 0))


def test_fp8_layer_close_to_dense_layer():
    """The FP8 restatement stays within quantisation noise of the unquantised layer."""
    torch.manual_seed(1)
    T, H, I, E, K = 12, 256, 128, 4, 2
    x = torch.randn(T, H).to(torch.bfloat16)
    logits = torch.randn(T, E)
    w13 = torch.randn(E, 2 * I, H) * 0.05
    w2 = torch.randn(E, H, I) * 0.05
    w13q, w13s = oracle.quantize_weight_ref(w13)
    w2q, w2s = oracle.quantize_weight_ref(w2)
    out = oracle.moe_fp8_ref(x, logits, w13q, w13s, w2q, w2s, K).float()
    dense = oracle.moe_dense_ref(x, logits, w13, w2, K)
    assert float((out - dense).abs().max() / dense.abs().max()) < 0.15


def test_weight_dequant_matches_hf_fp8dequantize_bit_exact():
    """Six tiles with six different scales: a transposed or mis-indexed scale grid cannot pass."""
    g = golden("fp8_weight_dequant.npz")
    q = torch.from_numpy(g["q"]).view(torch.float8_e4m3fn)
    w = oracle.dequant_weight(q, torch.from_numpy(g["scale_inv"]))
    np.testing.assert_array_equal(w.numpy(), g["w"])
    assert g["scale_inv"].shape == (1, 2, 3) and len(set(g["scale_inv"].reshape(-1).tolist())) == 6


@pytest.mark.parametrize("T,H,I,E,K,seed", [(64, 256, 128, 8, 2, 0), (32, 512, 256, 16, 4, 1)])
def test_fp32_until_quantised_stays_close_to_the_bf16_rounding_of_the_hf_experts(T, H, I, E, K, seed):
    """The kernels keep gate/up and h in fp32 until h is quantised; transformers FP8Experts.forward rounds
    them through bf16 (and multiplies the routing weight in bf16).  A bf16 rounding of h moves about one e4m3
    code in twenty to its neighbour (a 6 % step of that element), so the two forms sit about 2.5e-2 of the
    output's largest magnitude apart (1.7e-2 rms) at every size tried - the size of the e4m3 rounding of h
    itself, an order below the distance of either form to the unquantised layer (test above: up to 1.5e-1).
    Bounded at 4e-2; the kernels are held to 1e-2 against the form they implement."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    w13q, w13s = oracle.quantize_weight_ref(torch.randn(E, 2 * I, H, generator=g) * 0.05)
    w2q, w2s = oracle.quantize_weight_ref(torch.randn(E, H, I, generator=g) * 0.05)
    ours, parts = oracle.moe_fp8_ref(x, logits, w13q, w13s, w2q, w2s, K, return_parts=True)
    hf, hparts = oracle.moe_fp8_ref(x, logits, w13q, w13s, w2q, w2s, K, return_parts=True, hf_rounding=True)
    err = float((ours.float() - hf.float()).abs().max() / hf.float().abs().max())
    same_codes = float((parts["hq"].view(torch.uint8) == hparts["hq"].view(torch.uint8)).float().mean())
    print(f"fp32-until-quantised vs bf16-rounded: max err / max |out| = {err:.2e}, identical h codes {same_codes:.3f}")
    assert err < 4e-2
    assert same_codes > 0.9


def test_prompt_chunk_attention_matches_hf_eager_attention_with_causal_mask():
    """45 suffix tokens on 37 cached ones: pages gathered by the reference's blocks_to_dynamic_cache, attention
    by transformers eager_attention_forward under the causal mask."""
    g = golden("attn_prefill_d64.npz")
    t = lambda k: torch.from_numpy(g[k])
    out = oracle.paged_prefill_ref(t("q"), t("k_pool"), t("v_pool"), g["table_row"].tolist(), int(g["first_pos"]),
                                   float(g["scale"]))
    np.testing.assert_allclose(out.numpy(), g["out"], rtol=2e-5, atol=2e-6)
    # and row by row it is the decode oracle at that row's length
    row = 17
    one = oracle.paged_attn_ref(t("q")[row:row + 1], t("k_pool"), t("v_pool"), t("table_row").view(1, -1),
                                torch.tensor([int(g["first_pos"]) + row + 1]), float(g["scale"]))
    np.testing.assert_allclose(out[row].numpy(), one[0].numpy(), rtol=1e-5, atol=1e-6)
