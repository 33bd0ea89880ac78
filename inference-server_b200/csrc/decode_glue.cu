// Fused element-wise pieces between the decode step's GEMMs, attention and MoE.
//
// In the reference these run as dozens of small PyTorch ops per layer inside the
// model forward called at src/inference_server/backends/torch_backend.py:314-320
// (transformers Qwen3MoeDecoderLayer / Qwen3MoeAttention / Qwen3MoeRMSNorm):
//   add_rmsnorm        hidden = residual + delta;  normed = weight * (hidden /
//                      rms(hidden)) with the statistics in fp32, one pass.
//   qk_norm_rope_append  per-head RMSNorm of q and k, rotary embedding
//                      (rotate-half convention), q written contiguously for the
//                      attention kernel, k and v written straight into their page
//                      slot - the decode-time form of the page write at
//                      src/inference_server/kv_cache/cache_manager.py:185-214.
// Both are pure HBM/latency-bound byte shuffling with a little fp32 arithmetic.

#include "common.cuh"
#include "host.h"

namespace b200 {

__device__ __forceinline__ float block_sum(float v, float* sm) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = lane < nw ? sm[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// One CTA per row, 8 columns per thread.  x is updated in place when delta is given.
__global__ void add_rmsnorm_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                                   const __nv_bfloat16* __restrict__ weight, float eps, int H,
                                   __nv_bfloat16* __restrict__ out) {
  __shared__ float sm[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * H + threadIdx.x * 8;
  uint4 raw = *reinterpret_cast<const uint4*>(x + base);
  __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
  float f[8];
  if (delta != nullptr) {
    const uint4 draw = *reinterpret_cast<const uint4*>(delta + base);
    const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&draw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      h2[j] = __hadd2(h2[j], d2[j]);  // the residual add happens in bf16, as in the model
    }
    *reinterpret_cast<uint4*>(x + base) = raw;
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 p = __bfloat1622float2(h2[j]);
    f[2 * j] = p.x;
    f[2 * j + 1] = p.y;
    ss += p.x * p.x + p.y * p.y;
  }
  ss = block_sum(ss, sm);
  const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
  const uint4 wraw = *reinterpret_cast<const uint4*>(weight + threadIdx.x * 8);
  const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wraw);
  uint4 o;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // normalised value is rounded to bf16 before the weight multiply, as in the model
    const __nv_bfloat162 n = __floats2bfloat162_rn(f[2 * j] * inv, f[2 * j + 1] * inv);
    o2[j] = __hmul2(w2[j], n);
  }
  *reinterpret_cast<uint4*>(out + base) = o;
}

// One warp per (row, head) of the fused qkv projection output.
template <int D>
__global__ void __launch_bounds__(256)
qk_norm_rope_append_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ q_w,
                           const __nv_bfloat16* __restrict__ k_w, const __nv_bfloat16* __restrict__ cos_t,
                           const __nv_bfloat16* __restrict__ sin_t, const int* __restrict__ positions,
                           const int* __restrict__ block_table, __nv_bfloat16* __restrict__ q_out,
                           __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
                           int* __restrict__ err, int batch, int hq, int hkv, float eps, int page,
                           int num_blocks, int max_pages, int max_pos) {
  constexpr int PER = D / 32;  // elements per lane; lane holds d = lane + 32 * j
  const int heads = hq + 2 * hkv;
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= batch * heads) return;
  const int b = w / heads, h = w % heads;
  const int pos = positions[b];
  if (pos < 0 || pos >= max_pos || pos >= max_pages * page) {
    if (lane == 0) set_error(err, kErrDevBadCtxLen);
    return;
  }
  const __nv_bfloat16* src = qkv + (static_cast<size_t>(b) * heads + h) * D;
  float v[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) v[j] = __bfloat162float(src[lane + 32 * j]);

  const bool is_q = h < hq, is_k = !is_q && h < hq + hkv;
  if (is_q || is_k) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) ss += v[j] * v[j];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / static_cast<float>(D) + eps);
    const __nv_bfloat16* nw = is_q ? q_w : k_w;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const float n = __bfloat162float(__float2bfloat16(v[j] * inv));
      v[j] = __bfloat162float(__float2bfloat16(__bfloat162float(nw[lane + 32 * j]) * n));
    }
    // rotate-half: out[d] = x[d] * cos[d] + (d < D/2 ? -x[d + D/2] : x[d - D/2]) * sin[d]
    const __nv_bfloat16* c = cos_t + static_cast<size_t>(pos) * D;
    const __nv_bfloat16* s = sin_t + static_cast<size_t>(pos) * D;
    float r[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int d = lane + 32 * j;
      const int jp = (j + PER / 2) % PER;  // partner element lives in the same lane
      const float rot = j < PER / 2 ? -v[jp] : v[jp];
      r[j] = v[j] * __bfloat162float(c[d]) + rot * __bfloat162float(s[d]);
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) v[j] = r[j];
  }

  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + (static_cast<size_t>(b) * hq + h) * D;
  } else {
    const int id = block_table[static_cast<size_t>(b) * max_pages + pos / page];
    if (id < 0 || id >= num_blocks) {
      if (lane == 0) set_error(err, kErrDevBadBlockId);
      return;
    }
    const int kvh = is_k ? h - hq : h - hq - hkv;
    __nv_bfloat16* pool = is_k ? k_pool : v_pool;
    dst = pool + ((static_cast<size_t>(id) * hkv + kvh) * page + pos % page) * D;
  }
#pragma unroll
  for (int j = 0; j < PER; ++j) dst[lane + 32 * j] = __float2bfloat16(v[j]);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_add_rmsnorm(void* x, const void* delta, const void* weight, float eps,
                                int num_rows, int hidden, void* out, void* stream) {
  B200_REQUIRE(x && weight && out, "add_rmsnorm: null pointer");
  B200_REQUIRE(num_rows >= 0 && hidden > 0 && hidden % 256 == 0 && hidden <= 8192,
               "add_rmsnorm: hidden %d must be a multiple of 256 and <= 8192", hidden);
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) |
                 reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
               "add_rmsnorm: buffers must be 16-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  if (num_rows == 0) return 0;
  add_rmsnorm_kernel<<<num_rows, hidden / 8, 0, as_stream(stream)>>>(
      static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta),
      static_cast<const __nv_bfloat16*>(weight), eps, hidden, static_cast<__nv_bfloat16*>(out));
  B200_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int b200_qk_norm_rope_append(const void* qkv, const void* q_norm_weight,
                                        const void* k_norm_weight, const void* cos_table,
                                        const void* sin_table, const int32_t* positions,
                                        const int32_t* block_table, void* q_out, void* k_pool,
                                        void* v_pool, void* status_word, int batch, int num_q_heads,
                                        int num_kv_heads, int head_dim, float eps, int page_size,
                                        int num_blocks, int max_pages_per_seq, int max_positions,
                                        void* stream) {
  B200_REQUIRE(qkv && q_norm_weight && k_norm_weight && cos_table && sin_table && positions &&
                   block_table && q_out && k_pool && v_pool,
               "qk_norm_rope_append: null pointer");
  B200_REQUIRE(batch >= 0 && num_q_heads > 0 && num_kv_heads > 0 && page_size > 0 && num_blocks > 0 &&
                   max_pages_per_seq > 0 && max_positions > 0,
               "qk_norm_rope_append: non-positive dimension");
  B200_REQUIRE(head_dim == 64 || head_dim == 128, "qk_norm_rope_append: head_dim %d is not 64 or 128", head_dim);
  int rc = check_device(nullptr);
  if (rc) return rc;
  if (batch == 0) return 0;
  const int warps = batch * (num_q_heads + 2 * num_kv_heads);
  const int blocks = (warps + 7) / 8;
  cudaStream_t st = as_stream(stream);
#define B200_QK_ARGS                                                                                   \
  static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(q_norm_weight),            \
      static_cast<const __nv_bfloat16*>(k_norm_weight), static_cast<const __nv_bfloat16*>(cos_table),   \
      static_cast<const __nv_bfloat16*>(sin_table), positions, block_table,                            \
      static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_pool),                          \
      static_cast<__nv_bfloat16*>(v_pool), static_cast<int*>(status_word), batch, num_q_heads,          \
      num_kv_heads, eps, page_size, num_blocks, max_pages_per_seq, max_positions
  if (head_dim == 128)
    qk_norm_rope_append_kernel<128><<<blocks, 256, 0, st>>>(B200_QK_ARGS);
  else
    qk_norm_rope_append_kernel<64><<<blocks, 256, 0, st>>>(B200_QK_ARGS);
#undef B200_QK_ARGS
  B200_CUDA(cudaGetLastError());
  return 0;
}
