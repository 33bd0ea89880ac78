// Residual add + RMSNorm + router projection + top-k routing in one kernel (sm_100a).
//
// In the reference's model forward (src/inference_server/backends/torch_backend.py:314-320 ->
// transformers Qwen3MoeDecoderLayer / Qwen3MoeSparseMoeBlock) these are a residual add, the
// post-attention RMSNorm, the router's linear layer `gate` and Qwen3MoeTopKRouter (fp32 softmax,
// top-k, renormalisation): four dependent launches that move a few megabytes.  At decode sizes
// their cost is launch and memory latency, not bandwidth, so they are fused here:
//
//   x += delta (bf16);  h = weight * rmsnorm(x);  logits = h W_r^T (fp32);  ids, weights = top-k
//
//   grid   = (rows / 16) clusters of 8 CTAs.  A cluster owns 16 rows; CTA r of it owns the r-th
//            eighth of the hidden dimension, so the router matrix [E, H] (0.5 MiB at E = 128,
//            H = 2048, too much for one CTA to pull in time) is read as eight 64 KiB slices.
//   norm   = each CTA adds and squares its slice of the 16 rows; the eight partial sums of squares
//            meet through distributed shared memory (16 floats per CTA) and are added in rank order.
//   gemm   = [16 x H/8] x [H/8 x E] per CTA by mma.sync m16n8k16 (bf16 in, fp32 out): 134 MFLOP for
//            256 rows, far too little for the tcgen05 path to pay its set-up; warp w takes experts
//            16w..16w+15.  The eight partial logit tiles (16 x E fp32) meet through distributed
//            shared memory: CTA r sums rows 2r and 2r+1 in rank order.
//   route  = those two rows are routed by two warps exactly as moe_route_kernel does (selection on
//            the logits, ties to the lower expert id), on fp32 logits that never leave the chip.
// Everything is deterministic (fixed summation orders, no atomics).

#include "common.cuh"
#include "host.h"

namespace b200 {

constexpr int kRfRows = 16;      // rows per cluster
constexpr int kRfCluster = 8;    // CTAs per cluster = slices of the hidden dimension
constexpr int kRfThreads = 256;
constexpr int kRfMaxExperts = 128;

__device__ __forceinline__ uint32_t rf_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void rf_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float rf_ld_peer(const float* local, uint32_t rank) {
  uint32_t remote;
  asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote));
  return v;
}
__device__ __forceinline__ void rf_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

struct RouterFusedParams {
  __nv_bfloat16* x;             // [T, H] residual stream, updated in place when delta is given
  const __nv_bfloat16* delta;   // [T, H] or null
  const __nv_bfloat16* norm_w;  // [H]
  const __nv_bfloat16* router;  // [E, H]
  __nv_bfloat16* normed;        // [T, H]
  int* topk_ids;                // [T, K]
  float* topk_w;                // [T, K]
  float* logits_out;            // [T, E] or null
  const int* num_valid;         // device scalar or null
  float eps;
  int T, H, E, K, renorm;
};

__global__ void __launch_bounds__(kRfThreads, 1)
add_rmsnorm_route_kernel(const RouterFusedParams p) {
#ifdef B200_DEVICE_OK
  extern __shared__ __align__(16) uint8_t rf_smem[];
  const int cols = p.H / kRfCluster;       // this CTA's slice of the hidden dimension
  const int pitch = cols + 8;              // bf16 elements per smem row: 16 bytes of padding keep ldmatrix conflict-free
  __nv_bfloat16* a_tile = reinterpret_cast<__nv_bfloat16*>(rf_smem);   // [16][pitch]
  __nv_bfloat16* w_tile = a_tile + kRfRows * pitch;                     // [E][pitch]
  float* ss_part = reinterpret_cast<float*>(w_tile + static_cast<size_t>(p.E) * pitch);  // [16]
  float* inv_sm = ss_part + kRfRows;                                    // [16]
  float* lg_part = inv_sm + kRfRows;                                    // [16][E]
  float* lg_fin = lg_part + kRfRows * p.E;                              // [2][E]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = rf_cluster_rank();
  const int row0 = (static_cast<int>(blockIdx.x) / kRfCluster) * kRfRows;
  const int col0 = static_cast<int>(rank) * cols;

  // ---- the router slice [E][cols] starts flowing into shared memory right away
  {
    const int chunks_per_row = cols / 8;  // 16-byte pieces
    const int total = p.E * chunks_per_row;
    for (int i = tid; i < total; i += kRfThreads) {
      const int e = i / chunks_per_row, c = i - e * chunks_per_row;
      rf_cp_async16(smem_u32(w_tile + static_cast<size_t>(e) * pitch + c * 8),
                    p.router + static_cast<size_t>(e) * p.H + col0 + c * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  // The router matrix is a weight; the rows come from the kernels before this one.
  grid_dep_wait();
  grid_dep_launch();

  // ---- residual add, partial sums of squares: warp w owns rows 2w and 2w + 1
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = 2 * warp + rr, row = row0 + r;
    float ss = 0.f;
    for (int c = lane; c < cols / 8; c += 32) {
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (row < p.T) {
        const size_t off = static_cast<size_t>(row) * p.H + col0 + c * 8;
        raw = *reinterpret_cast<const uint4*>(p.x + off);
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
        if (p.delta != nullptr) {
          const uint4 draw = *reinterpret_cast<const uint4*>(p.delta + off);
          const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&draw);
#pragma unroll
          for (int j = 0; j < 4; ++j) h2[j] = __hadd2(h2[j], d2[j]);  // the residual add happens in bf16, as in the model
          *reinterpret_cast<uint4*>(p.x + off) = raw;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
      *reinterpret_cast<uint4*>(a_tile + r * pitch + c * 8) = raw;
    }
    ss = warp_sum(ss);
    if (lane == 0) ss_part[r] = ss;
  }
  __syncwarp();
  rf_cluster_sync();  // #1: every slice's partial sums are written
  if (tid < kRfRows) {
    float part[kRfCluster];
#pragma unroll
    for (int pr = 0; pr < kRfCluster; ++pr) part[pr] = rf_ld_peer(ss_part + tid, pr);
    float tot = 0.f;
#pragma unroll
    for (int pr = 0; pr < kRfCluster; ++pr) tot += part[pr];
    inv_sm[tid] = rsqrtf(tot / static_cast<float>(p.H) + p.eps);
  }
  __syncthreads();

  // ---- normalise: out = weight * bf16(x * inv); kept in shared memory as the A operand, written out as h
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = 2 * warp + rr, row = row0 + r;
    const float inv = inv_sm[r];
    for (int c = lane; c < cols / 8; c += 32) {
      uint4 raw = *reinterpret_cast<const uint4*>(a_tile + r * pitch + c * 8);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const uint4 wraw = *reinterpret_cast<const uint4*>(p.norm_w + col0 + c * 8);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wraw);
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h2[j]);
        o2[j] = __hmul2(w2[j], __floats2bfloat162_rn(f.x * inv, f.y * inv));
      }
      *reinterpret_cast<uint4*>(a_tile + r * pitch + c * 8) = o;
      if (row < p.T) *reinterpret_cast<uint4*>(p.normed + static_cast<size_t>(row) * p.H + col0 + c * 8) = o;
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // ---- partial logits of this slice: warp w takes experts 16w .. 16w + 15
  if (warp * 16 < p.E) {
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const int mat = lane >> 3, lr = lane & 7;
    const uint32_t a_addr = smem_u32(a_tile) + static_cast<uint32_t>(((mat & 1) * 8 + lr) * pitch * 2 + (mat >> 1) * 16);
    const uint32_t b_addr =
        smem_u32(w_tile) + static_cast<uint32_t>((warp * 16 + (mat >> 1) * 8 + lr) * pitch * 2 + (mat & 1) * 16);
    for (int ks = 0; ks < cols / 16; ++ks) {
      uint32_t a[4], b0, b1, b2, b3;
      ldmatrix_x4(a_addr + ks * 32, a[0], a[1], a[2], a[3]);
      ldmatrix_x4(b_addr + ks * 32, b0, b1, b2, b3);
      mma_bf16_16816(acc[0], a, b0, b1);
      mma_bf16_16816(acc[1], a, b2, b3);
    }
    const int gq = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int e = warp * 16 + nt * 8 + 2 * tq;
      lg_part[gq * p.E + e] = acc[nt][0];
      lg_part[gq * p.E + e + 1] = acc[nt][1];
      lg_part[(gq + 8) * p.E + e] = acc[nt][2];
      lg_part[(gq + 8) * p.E + e + 1] = acc[nt][3];
    }
  }
  __syncwarp();
  rf_cluster_sync();  // #2: every slice's partial logits are written

  // ---- CTA r finishes rows 2r and 2r + 1: slices summed in rank order
  {
    const int rl = tid >> 7, e = tid & 127;  // 256 threads = 2 rows x up to 128 experts
    if (e < p.E) {
      const int r = 2 * static_cast<int>(rank) + rl;
      float part[kRfCluster];
#pragma unroll
      for (int pr = 0; pr < kRfCluster; ++pr) part[pr] = rf_ld_peer(lg_part + r * p.E + e, pr);
      float tot = 0.f;
#pragma unroll
      for (int pr = 0; pr < kRfCluster; ++pr) tot += part[pr];
      lg_fin[rl * p.E + e] = tot;
      const int row = row0 + r;
      if (p.logits_out != nullptr && row < p.T) p.logits_out[static_cast<size_t>(row) * p.E + e] = tot;
    }
  }
  __syncthreads();

  // ---- top-k of the two rows (the arithmetic of moe_route_kernel)
  if (warp < 2) {
    const int row = row0 + 2 * static_cast<int>(rank) + warp;
    if (row < p.T) {
      const int E = p.E, K = p.K;
      if (p.num_valid != nullptr && row >= *p.num_valid) {
        if (lane < K) {
          p.topk_ids[static_cast<size_t>(row) * K + lane] = -1;
          p.topk_w[static_cast<size_t>(row) * K + lane] = 0.f;
        }
      } else {
        constexpr int kPer = kRfMaxExperts / 32;
        const float* lg = lg_fin + warp * E;
        float v[kPer];
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < kPer; ++j) {
          const int e = lane + 32 * j;
          v[j] = e < E ? lg[e] : -INFINITY;
          mx = fmaxf(mx, v[j]);
        }
        mx = warp_max(mx);
        float den = 0.f;
#pragma unroll
        for (int j = 0; j < kPer; ++j)
          if (lane + 32 * j < E) den += expf(v[j] - mx);
        den = warp_sum(den);
        unsigned taken = 0;
        float sel_sum = 0.f, my_p = 0.f;
        int my_id = 0;
        for (int k = 0; k < K; ++k) {
          float bv = -INFINITY;
          int be = 0x7fffffff;
#pragma unroll
          for (int j = 0; j < kPer; ++j) {
            const int e = lane + 32 * j;
            if (e < E && !((taken >> j) & 1u) && (be == 0x7fffffff || v[j] > bv)) {
              bv = v[j];
              be = e;
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            const bool better = oe != 0x7fffffff && (be == 0x7fffffff || ov > bv || (ov == bv && oe < be));
            if (better) {
              bv = ov;
              be = oe;
            }
          }
          if ((be & 31) == lane) taken |= 1u << (be >> 5);
          const float pr = expf(bv - mx);
          sel_sum += pr;
          if (lane == k) {
            my_p = pr;
            my_id = be;
          }
        }
        if (lane < K) {
          p.topk_ids[static_cast<size_t>(row) * K + lane] = my_id;
          p.topk_w[static_cast<size_t>(row) * K + lane] = my_p / (p.renorm ? sel_sum : den);
        }
      }
    }
  }
  __syncwarp();
  rf_cluster_sync();  // #3: nobody leaves while a peer may still read its shared memory
#endif
}

static size_t router_fused_smem(int H, int E) {
  const size_t pitch = static_cast<size_t>(H) / kRfCluster + 8;
  return (kRfRows + static_cast<size_t>(E)) * pitch * 2 + (2 * kRfRows + kRfRows * static_cast<size_t>(E) + 2 * E) * 4;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_add_rmsnorm_route_supported(int hidden, int num_experts, int top_k) {
  return hidden > 0 && hidden % (kRfCluster * 64) == 0 && num_experts > 0 && num_experts % 16 == 0 &&
         num_experts <= kRfMaxExperts && top_k > 0 && top_k <= 32 && top_k <= num_experts &&
         router_fused_smem(hidden, num_experts) <= 200 * 1024;
}

extern "C" int b200_add_rmsnorm_route(void* x, const void* delta, const void* norm_weight, float eps,
                                      const void* router_weight, int num_rows, int hidden, int num_experts,
                                      int top_k, int renormalize, const int32_t* num_valid_rows, void* normed_out,
                                      int32_t* topk_ids, float* topk_weights, float* logits_out, void* stream) {
  B200_REQUIRE(x && norm_weight && router_weight && normed_out && topk_ids && topk_weights,
               "add_rmsnorm_route: null pointer");
  B200_REQUIRE(num_rows >= 0, "add_rmsnorm_route: negative row count");
  B200_REQUIRE(b200_add_rmsnorm_route_supported(hidden, num_experts, top_k),
               "add_rmsnorm_route: hidden %d must be a multiple of 512, num_experts %d a multiple of 16 and at most "
               "%d, top_k %d at most min(32, num_experts)", hidden, num_experts, kRfMaxExperts, top_k);
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) |
                 reinterpret_cast<uintptr_t>(norm_weight) | reinterpret_cast<uintptr_t>(router_weight) |
                 reinterpret_cast<uintptr_t>(normed_out)) & 15) == 0,
               "add_rmsnorm_route: buffers must be 16-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  if (num_rows == 0) return 0;
  RouterFusedParams p{};
  p.x = static_cast<__nv_bfloat16*>(x);
  p.delta = static_cast<const __nv_bfloat16*>(delta);
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_weight);
  p.router = static_cast<const __nv_bfloat16*>(router_weight);
  p.normed = static_cast<__nv_bfloat16*>(normed_out);
  p.topk_ids = topk_ids;
  p.topk_w = topk_weights;
  p.logits_out = logits_out;
  p.num_valid = num_valid_rows;
  p.eps = eps;
  p.T = num_rows;
  p.H = hidden;
  p.E = num_experts;
  p.K = top_k;
  p.renorm = renormalize;
  const size_t smem = router_fused_smem(hidden, num_experts);
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&add_rmsnorm_route_kernel), static_cast<int>(smem));
  if (rc) return rc;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>((num_rows + kRfRows - 1) / kRfRows) * kRfCluster);
  cfg.blockDim = dim3(kRfThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kRfCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlapped_launch_enabled() ? 2 : 1;
  B200_CUDA(cudaLaunchKernelEx(&cfg, add_rmsnorm_route_kernel, p));
  return 0;
}
