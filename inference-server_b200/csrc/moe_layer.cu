// The FP8 MoE layer as one C-ABI call: route -> permute -> quantise+scatter ->
// gate/up GEMM -> down GEMM -> combine, all enqueued on the caller's stream into
// a caller-provided workspace.  Host code only; the kernels live in
// moe_route.cu and moe_gemm.cu.

#include "common.cuh"
#include "host.h"

namespace b200 {

static size_t up256(size_t v) { return (v + 255) & ~size_t(255); }

struct MoeCarve {
  size_t permute_ws, topk_ids, topk_w, sorted_pair, row_of_pair, expert_offsets, tiles, num_tiles,
      xq, xs, hq, hs, y, total;
};

static MoeCarve carve_moe(int T, int E, int K, int H, int I) {
  MoeCarve c;
  const size_t rows = static_cast<size_t>(T) * K;
  size_t off = 0;
  c.permute_ws = off;  // begins with the status word
  off += up256(b200_moe_permute_workspace_bytes(T, E, K));
  c.topk_ids = off;
  off += up256(rows * 4);
  c.topk_w = off;
  off += up256(rows * 4);
  c.sorted_pair = off;
  off += up256(rows * 4);
  c.row_of_pair = off;
  off += up256(rows * 4);
  c.expert_offsets = off;
  off += up256(static_cast<size_t>(E + 1) * 4);
  c.tiles = off;
  off += up256(static_cast<size_t>(b200_moe_max_tiles(T, E, K)) * 16);
  c.num_tiles = off;
  off += 256;
  c.xq = off;
  off += up256(rows * H);
  c.xs = off;
  off += up256(rows * (H / 128) * 4);
  c.hq = off;
  off += up256(rows * I);
  c.hs = off;
  off += up256(rows * (I / 128) * 4);
  c.y = off;
  off += up256(rows * H * 2);
  c.total = off;
  return c;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_moe_fp8_workspace_bytes(int num_tokens, int num_experts, int top_k,
                                               int hidden, int inter) {
  if (num_tokens < 0 || num_experts <= 0 || top_k <= 0 || hidden <= 0 || inter <= 0) return 256;
  return carve_moe(num_tokens, num_experts, top_k, hidden, inter).total;
}

// `routed_ids` / `routed_w`: routing that the caller has already done; the router step is then skipped.
static int moe_forward_impl(const void* x, const void* router_logits, int logits_dtype, const int32_t* routed_ids,
                            const float* routed_w, const void* w13,
                            const float* w13_scale_inv, const void* w2, const float* w2_scale_inv,
                            void* out, void* residual, const void* norm_weight, float eps, void* workspace,
                            size_t workspace_bytes, int num_tokens, int num_experts, int top_k, int hidden,
                            int inter, int renormalize, int weight_layout, void* stream) {
  B200_REQUIRE(x && (router_logits || (routed_ids && routed_w)) && w13 && w13_scale_inv && w2 && w2_scale_inv && out &&
                   workspace,
               "moe_fp8_forward: null pointer");
  B200_REQUIRE(num_tokens >= 0 && num_experts > 0 && top_k > 0 && hidden > 0 && inter > 0,
               "moe_fp8_forward: bad dimensions");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0,
               "moe_fp8_forward: workspace must be 256-byte aligned");
  const MoeCarve c = carve_moe(num_tokens, num_experts, top_k, hidden, inter);
  if (workspace_bytes < c.total) {
    set_detail("moe_fp8_forward: workspace %zu < required %zu", workspace_bytes, c.total);
    return -kErrWorkspace;
  }
  if (num_tokens == 0) return 0;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const int32_t* topk_ids = routed_ids ? routed_ids : reinterpret_cast<int32_t*>(ws + c.topk_ids);
  const float* topk_w = routed_w ? routed_w : reinterpret_cast<float*>(ws + c.topk_w);
  int32_t* sorted_pair = reinterpret_cast<int32_t*>(ws + c.sorted_pair);
  int32_t* row_of_pair = reinterpret_cast<int32_t*>(ws + c.row_of_pair);
  int32_t* expert_offsets = reinterpret_cast<int32_t*>(ws + c.expert_offsets);
  void* tiles = ws + c.tiles;
  int32_t* num_tiles = reinterpret_cast<int32_t*>(ws + c.num_tiles);
  void* status = ws;
  const int rows = num_tokens * top_k;

  int rc = 0;
  if (routed_ids == nullptr) {
    rc = b200_moe_route(router_logits, logits_dtype, num_tokens, num_experts, top_k, renormalize, nullptr,
                        reinterpret_cast<int32_t*>(ws + c.topk_ids), reinterpret_cast<float*>(ws + c.topk_w), stream);
    if (rc) return rc;
  }
  rc = b200_moe_permute_quant(topk_ids, x, num_tokens, num_experts, top_k, hidden, sorted_pair, row_of_pair,
                              expert_offsets, tiles, num_tiles, ws + c.xq, reinterpret_cast<float*>(ws + c.xs),
                              ws + c.permute_ws, b200_moe_permute_workspace_bytes(num_tokens, num_experts, top_k),
                              stream);
  if (rc) return rc;
  rc = b200_moe_fp8_gemm_gate_up(ws + c.xq, reinterpret_cast<float*>(ws + c.xs), w13, w13_scale_inv,
                                 tiles, num_tiles, ws + c.hq, reinterpret_cast<float*>(ws + c.hs),
                                 status, rows, num_experts, hidden, inter, weight_layout, stream);
  if (rc) return rc;
  rc = b200_moe_fp8_gemm_down(ws + c.hq, reinterpret_cast<float*>(ws + c.hs), w2, w2_scale_inv,
                              tiles, num_tiles, ws + c.y, nullptr, status, rows, num_experts, hidden, inter,
                              weight_layout, stream);
  if (rc) return rc;
  if (residual != nullptr)
    return b200_moe_combine_add_rmsnorm(ws + c.y, row_of_pair, topk_w, residual, norm_weight, eps, num_tokens,
                                        hidden, top_k, out, stream);
  return b200_moe_combine(ws + c.y, row_of_pair, topk_w, num_tokens, hidden, top_k, out, stream);
}

extern "C" int b200_moe_fp8_forward(const void* x, const void* router_logits, int logits_dtype,
                                    const void* w13, const float* w13_scale_inv, const void* w2,
                                    const float* w2_scale_inv, void* out, void* workspace,
                                    size_t workspace_bytes, int num_tokens, int num_experts,
                                    int top_k, int hidden, int inter, int renormalize,
                                    int weight_layout, void* stream) {
  return moe_forward_impl(x, router_logits, logits_dtype, nullptr, nullptr, w13, w13_scale_inv, w2, w2_scale_inv, out,
                          nullptr, nullptr, 0.f, workspace, workspace_bytes, num_tokens, num_experts, top_k, hidden, inter,
                          renormalize, weight_layout, stream);
}

extern "C" int b200_moe_fp8_forward_add_rmsnorm(const void* x, const void* router_logits, int logits_dtype,
                                                const void* w13, const float* w13_scale_inv, const void* w2,
                                                const float* w2_scale_inv, void* residual,
                                                const void* norm_weight, float eps, void* normed_out,
                                                void* workspace, size_t workspace_bytes, int num_tokens,
                                                int num_experts, int top_k, int hidden, int inter,
                                                int renormalize, int weight_layout, void* stream) {
  B200_REQUIRE(residual && norm_weight && normed_out, "moe_fp8_forward_add_rmsnorm: null pointer");
  return moe_forward_impl(x, router_logits, logits_dtype, nullptr, nullptr, w13, w13_scale_inv, w2, w2_scale_inv,
                          normed_out, residual, norm_weight, eps, workspace, workspace_bytes, num_tokens, num_experts,
                          top_k, hidden, inter, renormalize, weight_layout, stream);
}

extern "C" int b200_moe_fp8_routed_add_rmsnorm(const void* x, const int32_t* topk_ids, const float* topk_weights,
                                               const void* w13, const float* w13_scale_inv, const void* w2,
                                               const float* w2_scale_inv, void* residual, const void* norm_weight,
                                               float eps, void* normed_out, void* workspace, size_t workspace_bytes,
                                               int num_tokens, int num_experts, int top_k, int hidden, int inter,
                                               int weight_layout, void* stream) {
  B200_REQUIRE(topk_ids && topk_weights && residual && norm_weight && normed_out,
               "moe_fp8_routed_add_rmsnorm: null pointer");
  return moe_forward_impl(x, nullptr, 0, topk_ids, topk_weights, w13, w13_scale_inv, w2, w2_scale_inv, normed_out,
                          residual, norm_weight, eps, workspace, workspace_bytes, num_tokens, num_experts, top_k,
                          hidden, inter, 1, weight_layout, stream);
}
