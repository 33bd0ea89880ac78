// Paged GQA decode attention for sm_100a.
//
// Replaces, for one decode step, what the reference does with dense tensors:
// gather of the KV pages into a [B,H,S,D] cache
// (src/inference_server/kv_cache/hf_format.py:21-45), left padding
// (src/inference_server/backends/torch_backend.py:237-258) and the masked
// softmax(q K^T * scale) V with GQA head sharing inside the model forward
// (torch_backend.py:305-322).  Here the pools are read in place, in the
// reference layout [num_blocks, n_kv_heads, block_size, head_dim]
// (src/inference_server/kv_cache/block_manager.py:33-49).
//
// Main kernel (bf16 pools, page 16, head_dim 64 or 128, 1/2/4/8 kv heads):
//   grid  = (batch, max_splits), block = one consumer warp per kv head + 1
//           producer warp.  One CTA owns `split_tokens` consecutive tokens of one
//           sequence, for ALL kv heads: in the pool the kv heads of a page are
//           adjacent, so a page is one contiguous 16*Hkv*D*2-byte read for K and
//           one for V, which is what keeps the DRAM row buffers busy.
//   load  = the producer warp looks the page id up in the block table and issues
//           one TMA box (16*Hkv rows x 128 bytes, 128-byte swizzle) per 128-byte
//           column half for K and for V into a ring of one-page stages; stage
//           hand-over is by mbarrier (full: transaction bytes, empty: Hkv warps).
//   math  = consumer warp w owns kv head w: S = Q K^T with mma.sync m16n8k16
//           (rows = the <=16 query heads of the kv group), online softmax in
//           fp32 with quad shuffles, O += P V.  Warps never exchange data.
//   out   = a sequence that fits one split is normalised and written as bf16
//           straight from registers.  Otherwise each warp writes one fp32
//           partial (o, m, l) per (sequence, q head, split) and a second, small
//           kernel folds the splits in split order and writes bf16.
// The kernel is HBM-bound: per token and kv head it reads 2*D*2 bytes once.
//
// Generic kernel: any head_dim <= 256, any page size, fp32 or bf16 pools, no
// split, fp32 arithmetic throughout.  It serves shapes the main kernel does not
// (the tiny fp32 parity model) and is not tuned.

#include <mutex>

#include "common.cuh"
#include "host.h"

namespace b200 {

constexpr int kPage = 16;               // tokens per page in the main kernel
constexpr int kBoxBytes = kPage * 128;  // one TMA box: 16 rows x 128 bytes

// D: head_dim.  HKV: kv heads = consumer warps.  STAGES: pipeline depth in pages.
// CTAS: CTAs resident per SM the launch bounds aim for.
template <int D, int HKV, int STAGES, int CTAS>
struct AttnCfg {
  static constexpr int kThreads = (HKV + 1) * 32;
  static constexpr int kHalves = D / 64;                     // 128-byte column halves per row
  static constexpr int kHeadBytes = kBoxBytes;               // one head's 16 rows x 128 B inside a box
  static constexpr int kBoxAll = HKV * kBoxBytes;            // one TMA box: all kv heads of a page half
  static constexpr int kStageBytes = 2 * kHalves * kBoxAll;  // K halves then V halves
  static constexpr int kRingBytes = STAGES * kStageBytes;
  static constexpr int kSmemBytes = kRingBytes + 1024 /* alignment slack */ + 16 * STAGES /* barriers */;
};

// PAIRS: two rows per CTA - batch rows 2i and 2i+1, which must share block_table row 2i (two consecutive tokens
// of one prompt).  The second row rides in the upper eight rows of the m16 MMA tile, which a kv group of up to
// eight query heads leaves idle, so a prompt chunk reads every page half as often.
template <int D, int HKV, int STAGES, int CTAS, bool PAIRS = false>
__global__ void __launch_bounds__((HKV + 1) * 32, CTAS)
paged_attn_decode_kernel(const __grid_constant__ CUtensorMap k_map,
                         const __grid_constant__ CUtensorMap v_map,
                         const __nv_bfloat16* __restrict__ q,
                         const int* __restrict__ block_table,
                         const int* __restrict__ ctx_lens,
                         float* __restrict__ part_o, float2* __restrict__ part_ml,
                         __nv_bfloat16* __restrict__ out,
                         int* __restrict__ err, int batch, int num_q_heads, int num_blocks, int max_pages,
                         int split_tokens, int max_splits, float scale_log2) {
#ifdef B200_DEVICE_OK
  grid_dep_wait();    // the context lengths, the query rows and the new K/V rows come from the kernels before
  grid_dep_launch();
  using Cfg = AttnCfg<D, HKV, STAGES, CTAS>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = ring + Cfg::kRingBytes;  // full[STAGES], empty[STAGES]

  const int b = PAIRS ? 2 * blockIdx.x : blockIdx.x, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = num_q_heads / HKV;
  const bool has1 = PAIRS && b + 1 < batch;  // the pair's second row exists

  int L = ctx_lens[b];
  if (L < 0 || L > max_pages * kPage) {
    if (threadIdx.x == 0) set_error(err, kErrDevBadCtxLen);
    L = L < 0 ? 0 : max_pages * kPage;
  }
  int L0 = L, L1 = 0;  // PAIRS: lengths of the two rows; L becomes the longer one
  if (PAIRS) {
    if (has1) {
      L1 = ctx_lens[b + 1];
      if (L1 < 0 || L1 > max_pages * kPage) {
        if (threadIdx.x == 0) set_error(err, kErrDevBadCtxLen);
        L1 = L1 < 0 ? 0 : max_pages * kPage;
      }
    }
    if (split == 0) {  // a row with no context attends to nothing: zeros
      if (L0 == 0)
        for (int i = threadIdx.x; i < num_q_heads * D; i += blockDim.x)
          out[static_cast<size_t>(b) * num_q_heads * D + i] = __float2bfloat16(0.f);
      if (has1 && L1 == 0)
        for (int i = threadIdx.x; i < num_q_heads * D; i += blockDim.x)
          out[static_cast<size_t>(b + 1) * num_q_heads * D + i] = __float2bfloat16(0.f);
    }
    L = max(L0, L1);
  }
  const int start = split * split_tokens;
  if (start >= L) {  // uniform for the whole CTA
    if (!PAIRS && L == 0 && split == 0)  // a row with no context attends to nothing: zeros
      for (int i = threadIdx.x; i < num_q_heads * D; i += blockDim.x)
        out[static_cast<size_t>(b) * num_q_heads * D + i] = __float2bfloat16(0.f);
    return;
  }
  const int end = min(L, start + split_tokens);
  const int npages = (end - start + kPage - 1) / kPage;
  const int first_page = start / kPage;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bars + 8 * s, 1);
      mbar_init(bars + 8 * (STAGES + s), HKV);
    }
    fence_mbar_init();
    fence_proxy_async();
  }
  __syncthreads();

  if (warp == HKV) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
    }
    const int* table_row = block_table + static_cast<size_t>(b) * max_pages + first_page;
    // lane -> (K or V, column half); one box each
    const int lkv = lane / Cfg::kHalves, lh = lane % Cfg::kHalves;
    const bool issuer = lane < 2 * Cfg::kHalves;
    // page ids of this split, 32 at a time, one per lane
    int ids = 0;
    for (int i = 0; i < npages; ++i) {
      if ((i & 31) == 0) {
        ids = i + lane < npages ? table_row[i + lane] : 0;
        if (ids < 0 || ids >= num_blocks) {
          set_error(err, kErrDevBadBlockId);
          ids = 0;
        }
      }
      const int id = __shfl_sync(0xffffffffu, ids, i & 31);
      const int slot = i % STAGES;
      const uint32_t phase = (i / STAGES) & 1;
      if (!mbar_wait(bars + 8 * (STAGES + slot), phase ^ 1, err)) break;
      if (lane == 0) mbar_arrive_expect_tx(bars + 8 * slot, Cfg::kStageBytes);
      __syncwarp();
      if (issuer) {
        const uint32_t dst = ring + slot * Cfg::kStageBytes + (lkv * Cfg::kHalves + lh) * Cfg::kBoxAll;
        tma_load_2d(dst, lkv ? &v_map : &k_map, bars + 8 * slot, lh * 64, id * (HKV * kPage));
      }
    }
    return;
  }

  // --------------------------------------------------------------- consumers --
  const int kvh = warp;      // this warp's kv head
  const int gq = lane >> 2;  // fragment row (query head inside the kv group)
  const int tq = lane & 3;
  const bool hi_rows = PAIRS ? has1 : group > 8;
  // upper eight tile rows: heads 8.. of the same row, or (PAIRS) heads 0..7 of the pair's second row
  const bool hi_ok = PAIRS ? (has1 && gq < group) : gq + 8 < group;

  // Q fragments for every 16-wide slice of head_dim (A operand, rows = heads).
  uint32_t qa[D / 16][4];
  {
    const __nv_bfloat16* qb = q + (static_cast<size_t>(b) * num_q_heads + kvh * group) * D;
    const __nv_bfloat16* qhi = PAIRS ? qb + static_cast<size_t>(num_q_heads) * D + static_cast<size_t>(gq) * D
                                     : qb + static_cast<size_t>(gq + 8) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int d0 = ks * 16 + 2 * tq;
      const uint32_t* r0 = reinterpret_cast<const uint32_t*>(qb + static_cast<size_t>(gq) * D + d0);
      const uint32_t* r1 = reinterpret_cast<const uint32_t*>(qhi + d0);
      qa[ks][0] = gq < group ? __ldg(r0) : 0u;
      qa[ks][1] = hi_ok ? __ldg(r1) : 0u;
      qa[ks][2] = gq < group ? __ldg(r0 + 4) : 0u;
      qa[ks][3] = hi_ok ? __ldg(r1 + 4) : 0u;
    }
  }

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // ldmatrix lane roles
  const int lj = lane >> 3, lr = lane & 7;
  const int k_tok = (lj >> 1) * 8 + lr;  // K: matrices 0,1 -> tokens 0-7; 2,3 -> tokens 8-15
  const int k_sub = lj & 1;              //    matrices 0,2 -> low 8 of the k-slice; 1,3 -> high 8
  const int v_tok = (lj & 1) * 8 + lr;   // V: matrices 0,2 -> tokens 0-7; 1,3 -> tokens 8-15
  const int v_sub = lj >> 1;             //    matrices 0,1 -> first n-tile; 2,3 -> second n-tile

  bool alive = true;
  for (int i = 0; i < npages && alive; ++i) {
    const int slot = i % STAGES;
    const uint32_t phase = (i / STAGES) & 1;
    alive = mbar_wait(bars + 8 * slot, phase, err);
    if (alive) {
      const uint32_t kbase = ring + slot * Cfg::kStageBytes + kvh * Cfg::kHeadBytes;
      const uint32_t vbase = kbase + Cfg::kHalves * Cfg::kBoxAll;

      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int cidx = ks * 2 + k_sub;
        uint32_t b00, b01, b10, b11;
        ldmatrix_x4(kbase + (cidx >> 3) * Cfg::kBoxAll + swz128(k_tok, cidx & 7), b00, b01, b10, b11);
        mma_bf16_16816(s0, qa[ks], b00, b01);
        mma_bf16_16816(s1, qa[ks], b10, b11);
      }

      const int tok0 = start + i * kPage + 2 * tq;  // token of s0[0]; s0[1] is +1, s1[*] is +8
      if (PAIRS) {
        // the two rows end at different tokens (a prompt's causal mask); the shorter one may even end before
        // this page starts, then everything of it is masked here
        if (start + i * kPage + kPage > min(L0, L1)) {
          if (tok0 >= L0) s0[0] = -INFINITY;
          if (tok0 + 1 >= L0) s0[1] = -INFINITY;
          if (tok0 + 8 >= L0) s1[0] = -INFINITY;
          if (tok0 + 9 >= L0) s1[1] = -INFINITY;
          if (tok0 >= L1) s0[2] = -INFINITY;
          if (tok0 + 1 >= L1) s0[3] = -INFINITY;
          if (tok0 + 8 >= L1) s1[2] = -INFINITY;
          if (tok0 + 9 >= L1) s1[3] = -INFINITY;
        }
      } else if (start + i * kPage + kPage > L) {
        if (tok0 >= L) s0[0] = s0[2] = -INFINITY;
        if (tok0 + 1 >= L) s0[1] = s0[3] = -INFINITY;
        if (tok0 + 8 >= L) s1[0] = s1[2] = -INFINITY;
        if (tok0 + 9 >= L) s1[1] = s1[3] = -INFINITY;
      }

      // online softmax, log2 domain; rows gq (index 0,1) and gq + 8 (index 2,3)
      float mx0 = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      // A PAIRS row that has seen nothing yet (everything masked so far) keeps m = -inf; its exponentials then
      // take 0 as their reference point and come out 0 instead of NaN.
      const float mnew0 = fmaxf(m0, mx0 * scale_log2);
      const float mn0 = (PAIRS && mnew0 == -INFINITY) ? 0.f : mnew0;
      const float a0 = exp2f(m0 - mn0);
      m0 = mnew0;
      const float p00 = exp2f(s0[0] * scale_log2 - mn0), p01 = exp2f(s0[1] * scale_log2 - mn0);
      const float p10 = exp2f(s1[0] * scale_log2 - mn0), p11 = exp2f(s1[1] * scale_log2 - mn0);
      l0 = l0 * a0 + (p00 + p01) + (p10 + p11);
      float a1 = 1.f, p02 = 0.f, p03 = 0.f, p12 = 0.f, p13 = 0.f;
      if (hi_rows) {
        float mx1 = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mnew1 = fmaxf(m1, mx1 * scale_log2);
        const float mn1 = (PAIRS && mnew1 == -INFINITY) ? 0.f : mnew1;
        a1 = exp2f(m1 - mn1);
        m1 = mnew1;
        p02 = exp2f(s0[2] * scale_log2 - mn1);
        p03 = exp2f(s0[3] * scale_log2 - mn1);
        p12 = exp2f(s1[2] * scale_log2 - mn1);
        p13 = exp2f(s1[3] * scale_log2 - mn1);
        l1 = l1 * a1 + (p02 + p03) + (p12 + p13);
      }
      uint32_t pa[4];
      pa[0] = pack_bf16x2(p00, p01);
      pa[1] = pack_bf16x2(p02, p03);
      pa[2] = pack_bf16x2(p10, p11);
      pa[3] = pack_bf16x2(p12, p13);

      const bool rescale = __any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f);
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
        if (rescale) {
          o[2 * np][0] *= a0;
          o[2 * np][1] *= a0;
          o[2 * np + 1][0] *= a0;
          o[2 * np + 1][1] *= a0;
          o[2 * np][2] *= a1;
          o[2 * np][3] *= a1;
          o[2 * np + 1][2] *= a1;
          o[2 * np + 1][3] *= a1;
        }
        const int cidx = np * 2 + v_sub;
        uint32_t v0, v1, v2, v3;
        ldmatrix_x4_trans(vbase + (cidx >> 3) * Cfg::kBoxAll + swz128(v_tok, cidx & 7), v0, v1, v2, v3);
        mma_bf16_16816(o[2 * np], pa, v0, v1);
        mma_bf16_16816(o[2 * np + 1], pa, v2, v3);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bars + 8 * (STAGES + slot));
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  if (PAIRS) {
    // each of the two rows has its own number of splits; a row takes part in this split only if it has tokens here
    const int n0 = (L0 + split_tokens - 1) / split_tokens, n1 = (L1 + split_tokens - 1) / split_tokens;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int nr = half ? n1 : n0;
      const bool ok = half ? hi_ok : gq < group;
      if (!ok || split >= nr) continue;
      const size_t qrow = (static_cast<size_t>(b + half) * num_q_heads + kvh * group + gq);
      const float lr = half ? l1 : l0, mr = half ? m1 : m0;
      if (nr == 1) {
        const float inv = 1.f / lr;
        __nv_bfloat16* od = out + qrow * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
          *reinterpret_cast<uint32_t*>(od + n * 8 + 2 * tq) =
              pack_bf16x2(o[n][2 * half] * inv, o[n][2 * half + 1] * inv);
      } else {
        const size_t prow = qrow * max_splits + split;
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
          *reinterpret_cast<float2*>(part_o + prow * D + n * 8 + 2 * tq) = make_float2(o[n][2 * half], o[n][2 * half + 1]);
        if (tq == 0) part_ml[prow] = make_float2(mr, lr);
      }
    }
    return;
  }

  const int nsplits = (L + split_tokens - 1) / split_tokens;  // CTAs working on this sequence
  if (nsplits == 1) {
    // The whole sequence was this CTA's: normalise and write the result, no partials.
    const float i0 = 1.f / l0, i1 = hi_rows ? 1.f / l1 : 0.f;
    __nv_bfloat16* o0 = out + (static_cast<size_t>(b) * num_q_heads + kvh * group + gq) * D;
    __nv_bfloat16* o1 = o0 + static_cast<size_t>(8) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      const int d = n * 8 + 2 * tq;
      if (gq < group) *reinterpret_cast<uint32_t*>(o0 + d) = pack_bf16x2(o[n][0] * i0, o[n][1] * i0);
      if (gq + 8 < group) *reinterpret_cast<uint32_t*>(o1 + d) = pack_bf16x2(o[n][2] * i1, o[n][3] * i1);
    }
    return;
  }

  // Each warp owns its kv head's query rows: write the split partial directly.
  const size_t row0 = (static_cast<size_t>(b) * num_q_heads + kvh * group + gq) * max_splits + split;
  const size_t row1 = row0 + static_cast<size_t>(8) * max_splits;
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    const int d = n * 8 + 2 * tq;
    if (gq < group) *reinterpret_cast<float2*>(part_o + row0 * D + d) = make_float2(o[n][0], o[n][1]);
    if (gq + 8 < group) *reinterpret_cast<float2*>(part_o + row1 * D + d) = make_float2(o[n][2], o[n][3]);
  }
  if (tq == 0) {
    if (gq < group) part_ml[row0] = make_float2(m0, l0);
    if (gq + 8 < group) part_ml[row1] = make_float2(m1, l1);
  }

#endif
}

// Folds the per-split partials of one (sequence, q head) in split order: one warp
// per row; lanes first cover the splits (max and normaliser by shuffles), then
// head_dim in float4 pieces with the per-split weights broadcast from registers.
// Sequences with a single split were already written by the main kernel.
template <int D>
__global__ void __launch_bounds__(128)
paged_attn_reduce_kernel(const float* __restrict__ part_o, const float2* __restrict__ part_ml,
                         const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out,
                         int rows_total, int num_q_heads, int max_splits, int split_tokens, int max_ctx) {
  grid_dep_wait();
  grid_dep_launch();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows_total) return;
  const int b = row / num_q_heads;
  int L = ctx_lens[b];
  L = L < 0 ? 0 : (L > max_ctx ? max_ctx : L);
  const int n = (L + split_tokens - 1) / split_tokens;
  if (n <= 1) return;
  const size_t base = static_cast<size_t>(row) * max_splits;
  constexpr int V = D / 32;  // floats per lane
  // The first eight partial rows (all of them at the usual split counts) are asked for before anything else:
  // their addresses need only n, and the kernel is bound by the latency of its loads, not by their volume.
  float pre[8][V];
  const int npre = min(n, 8);
#pragma unroll
  for (int u = 0; u < 8; ++u)
    if (u < npre)
#pragma unroll
      for (int j = 0; j < V; ++j) pre[u][j] = part_o[(base + u) * D + lane * V + j];
  float mmax = -INFINITY;
  for (int s0 = 0; s0 < n; s0 += 32) {
    const float m = s0 + lane < n ? part_ml[base + s0 + lane].x : -INFINITY;
    mmax = fmaxf(mmax, warp_max(m));
  }
  float den = 0.f;
  float acc[V];
#pragma unroll
  for (int j = 0; j < V; ++j) acc[j] = 0.f;
  for (int s0 = 0; s0 < n; s0 += 32) {
    float w = 0.f;
    if (s0 + lane < n) {
      const float2 ml = part_ml[base + s0 + lane];
      w = exp2f(ml.x - mmax);
      den += w * ml.y;
    }
    const int cnt = min(32, n - s0);
    int s = 0;
    if (s0 == 0) {  // the rows fetched above, in split order like the rest
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (u < npre) {
          const float wu = __shfl_sync(0xffffffffu, w, u);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += wu * pre[u][j];
        }
      s = npre;
    }
    for (; s + 4 <= cnt; s += 4) {
      float v[4][V];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < V; ++j) v[u][j] = part_o[(base + s0 + s + u) * D + lane * V + j];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float wu = __shfl_sync(0xffffffffu, w, s + u);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += wu * v[u][j];
      }
    }
    for (; s < cnt; ++s) {
      const float wu = __shfl_sync(0xffffffffu, w, s);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += wu * part_o[(base + s0 + s) * D + lane * V + j];
    }
  }
  den = warp_sum(den);
  const float inv = 1.f / den;
  __nv_bfloat16* dst = out + static_cast<size_t>(row) * D + lane * V;
#pragma unroll
  for (int j = 0; j < V; j += 2)
    *reinterpret_cast<uint32_t*>(dst + j) = pack_bf16x2(acc[j] * inv, acc[j + 1] * inv);
}

// ------------------------------------------------------------ generic path --
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

constexpr int kGenWarps = 4;
constexpr int kGenMaxPerLane = 8;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(kGenWarps * 32)
paged_attn_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                          const T* __restrict__ v_pool, const int* __restrict__ block_table,
                          const int* __restrict__ ctx_lens, T* __restrict__ out,
                          int* __restrict__ err, int num_q_heads, int num_kv_heads, int D, int page,
                          int num_blocks, int max_pages, float scale) {
  __shared__ float o_sm[kGenWarps][256];
  __shared__ float m_sm[kGenWarps], l_sm[kGenWarps];
  const int h = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = h / (num_q_heads / num_kv_heads);
  int L = ctx_lens[b];
  if (L < 0 || L > max_pages * page) {
    if (threadIdx.x == 0) set_error(err, kErrDevBadCtxLen);
    L = L < 0 ? 0 : max_pages * page;
  }
  float qr[kGenMaxPerLane], acc[kGenMaxPerLane];
#pragma unroll
  for (int j = 0; j < kGenMaxPerLane; ++j) {
    const int d = lane + 32 * j;
    qr[j] = d < D ? to_f32<T>(q[(static_cast<size_t>(b) * num_q_heads + h) * D + d]) : 0.f;
    acc[j] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int tok = warp; tok < L; tok += kGenWarps) {
    int id = block_table[static_cast<size_t>(b) * max_pages + tok / page];
    if (id < 0 || id >= num_blocks) {
      set_error(err, kErrDevBadBlockId);
      id = 0;
    }
    const size_t base = ((static_cast<size_t>(id) * num_kv_heads + kvh) * page + tok % page) * D;
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < kGenMaxPerLane; ++j) {
      const int d = lane + 32 * j;
      if (d < D) dot += qr[j] * to_f32<T>(k_pool[base + d]);
    }
    dot = warp_sum(dot) * scale;
    const float mn = fmaxf(m, dot);
    const float a = expf(m - mn), p = expf(dot - mn);
    m = mn;
    l = l * a + p;
#pragma unroll
    for (int j = 0; j < kGenMaxPerLane; ++j) {
      const int d = lane + 32 * j;
      if (d < D) acc[j] = acc[j] * a + p * to_f32<T>(v_pool[base + d]);
    }
  }
#pragma unroll
  for (int j = 0; j < kGenMaxPerLane; ++j) {
    const int d = lane + 32 * j;
    if (d < D) o_sm[warp][d] = acc[j];
  }
  if (lane == 0) {
    m_sm[warp] = m;
    l_sm[warp] = l;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float mmax = -INFINITY;
    for (int w = 0; w < kGenWarps; ++w) mmax = fmaxf(mmax, m_sm[w]);
    float num = 0.f, den = 0.f;
    for (int w = 0; w < kGenWarps; ++w) {
      const float wgt = m_sm[w] == -INFINITY ? 0.f : expf(m_sm[w] - mmax);
      num += wgt * o_sm[w][d];
      den += wgt * l_sm[w];
    }
    out[(static_cast<size_t>(b) * num_q_heads + h) * D + d] = from_f32<T>(den > 0.f ? num / den : 0.f);
  }
}

// Writes this step's K and V rows ([B, n_kv_heads, D]) into their page slots:
// the decode-time counterpart of the reference's prompt-only page write
// (src/inference_server/kv_cache/cache_manager.py:185-214).
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new,
                                 T* __restrict__ k_pool, T* __restrict__ v_pool,
                                 const int* __restrict__ block_table,
                                 const int* __restrict__ positions, int* __restrict__ err,
                                 int num_kv_heads, int D, int page, int num_blocks,
                                 int max_pages) {
  const int b = blockIdx.x;
  const int pos = positions[b];
  if (pos < 0 || pos >= max_pages * page) {
    if (threadIdx.x == 0) set_error(err, kErrDevBadCtxLen);
    return;
  }
  const int id = block_table[static_cast<size_t>(b) * max_pages + pos / page];
  if (id < 0 || id >= num_blocks) {
    if (threadIdx.x == 0) set_error(err, kErrDevBadBlockId);
    return;
  }
  const int slot = pos % page;
  for (int i = threadIdx.x; i < num_kv_heads * D; i += blockDim.x) {
    const int h = i / D, d = i % D;
    const size_t dst = ((static_cast<size_t>(id) * num_kv_heads + h) * page + slot) * D + d;
    const size_t src = static_cast<size_t>(b) * num_kv_heads * D + i;
    k_pool[dst] = k_new[src];
    v_pool[dst] = v_new[src];
  }
}

// ------------------------------------------------------------------ launch --
struct AttnWorkspace {
  int* err;
  float2* ml;
  float* o;
  size_t bytes;
};

static int max_splits_of(int max_pages, int page, int split_tokens) {
  return (max_pages * page + split_tokens - 1) / split_tokens;
}

static AttnWorkspace carve(void* ws, int batch, int hq, int D, int max_splits) {
  AttnWorkspace w;
  uint8_t* p = static_cast<uint8_t*>(ws);
  w.err = reinterpret_cast<int*>(p);
  size_t off = 256;
  w.ml = reinterpret_cast<float2*>(p + off);
  off += (static_cast<size_t>(batch) * hq * max_splits * sizeof(float2) + 255) & ~size_t(255);
  w.o = reinterpret_cast<float*>(p + off);
  off += static_cast<size_t>(batch) * hq * max_splits * D * sizeof(float);
  w.bytes = off;
  return w;
}

template <int D, int HKV, int STAGES, int CTAS, bool PAIRS = false>
static int launch_main(const void* q, const void* k_pool, const void* v_pool,
                       const int* block_table, const int* ctx_lens, void* out,
                       const AttnWorkspace& w, int batch, int hq, int num_blocks, int max_pages,
                       float scale, int split_tokens, int max_splits, cudaStream_t stream) {
  using Cfg = AttnCfg<D, HKV, STAGES, CTAS>;
  CUtensorMap kmap, vmap;
  const uint64_t rows = static_cast<uint64_t>(num_blocks) * HKV * kPage;
  int rc = get_tensor_map_2d(k_pool, rows, D, 2, HKV * kPage, 64, &kmap);
  if (rc) return rc;
  rc = get_tensor_map_2d(v_pool, rows, D, 2, HKV * kPage, 64, &vmap);
  if (rc) return rc;
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&paged_attn_decode_kernel<D, HKV, STAGES, CTAS, PAIRS>),
                           Cfg::kSmemBytes);
  if (rc) return rc;
  dim3 grid(PAIRS ? (batch + 1) / 2 : batch, max_splits);
  const float scale_log2 = scale * 1.4426950408889634f;
  B200_CUDA(launch_overlapped(paged_attn_decode_kernel<D, HKV, STAGES, CTAS, PAIRS>, grid, dim3(Cfg::kThreads),
                              Cfg::kSmemBytes, stream, kmap, vmap, static_cast<const __nv_bfloat16*>(q), block_table,
                              ctx_lens, w.o, w.ml, static_cast<__nv_bfloat16*>(out), w.err, batch, hq, num_blocks,
                              max_pages, split_tokens, max_splits, scale_log2));
  if (max_splits > 1) {
    const int rows = batch * hq;
    B200_CUDA(launch_overlapped(paged_attn_reduce_kernel<D>, dim3((rows + 3) / 4), dim3(128), 0, stream, w.o, w.ml,
                                ctx_lens, static_cast<__nv_bfloat16*>(out), rows, hq, max_splits, split_tokens,
                                max_pages * kPage));
  }
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_paged_attn_workspace_bytes(int batch, int num_q_heads, int head_dim,
                                                  int max_pages_per_seq, int page_size,
                                                  int split_tokens) {
  if (batch <= 0 || num_q_heads <= 0 || head_dim <= 0 || max_pages_per_seq <= 0 || page_size <= 0 ||
      split_tokens <= 0)
    return 256;
  const int ms = max_splits_of(max_pages_per_seq, page_size, split_tokens);
  return carve(nullptr, batch, num_q_heads, head_dim, ms).bytes;
}

extern "C" int b200_paged_attn_decode(const void* q, const void* k_pool, const void* v_pool,
                                      const int32_t* block_table, const int32_t* ctx_lens,
                                      void* out, void* workspace, size_t workspace_bytes, int batch,
                                      int num_q_heads, int num_kv_heads, int head_dim,
                                      int page_size, int num_blocks, int max_pages_per_seq,
                                      float scale, int split_tokens, int dtype, void* stream) {
  B200_REQUIRE(q && k_pool && v_pool && block_table && ctx_lens && out && workspace,
               "paged_attn_decode: null pointer");
  B200_REQUIRE(batch > 0 && num_q_heads > 0 && num_kv_heads > 0 && num_blocks > 0 &&
                   max_pages_per_seq > 0 && page_size > 0,
               "paged_attn_decode: non-positive dimension");
  B200_REQUIRE(num_q_heads % num_kv_heads == 0, "paged_attn_decode: q heads %d not a multiple of kv heads %d",
               num_q_heads, num_kv_heads);
  B200_REQUIRE(head_dim > 0 && head_dim <= 256, "paged_attn_decode: head_dim %d outside (0, 256]", head_dim);
  B200_REQUIRE(dtype == 0 || dtype == 1, "paged_attn_decode: dtype %d is neither 0 (bf16) nor 1 (f32)", dtype);
  B200_REQUIRE(workspace_bytes >= 256, "paged_attn_decode: workspace smaller than the status word block");
  int dev = 0;
  int rc = check_device(&dev);
  if (rc) return rc;
  cudaStream_t st = as_stream(stream);
  const int group = num_q_heads / num_kv_heads;
  const bool fast = dtype == 0 && page_size == kPage && (head_dim == 64 || head_dim == 128) &&
                    group <= 16 && split_tokens > 0 &&
                    (num_kv_heads == 1 || num_kv_heads == 2 || num_kv_heads == 4 || num_kv_heads == 8);
  if (fast) {
    B200_REQUIRE(split_tokens % kPage == 0, "paged_attn_decode: split_tokens %d not a multiple of %d",
                 split_tokens, kPage);
    B200_REQUIRE((reinterpret_cast<uintptr_t>(k_pool) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(v_pool) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(q) & 3) == 0,
                 "paged_attn_decode: pools must be 16-byte aligned");
    const int ms = max_splits_of(max_pages_per_seq, page_size, split_tokens);
    B200_REQUIRE(ms <= 65535, "paged_attn_decode: grid too large");
    AttnWorkspace w = carve(workspace, batch, num_q_heads, head_dim, ms);
    if (workspace_bytes < w.bytes) {
      set_detail("paged_attn_decode: workspace %zu < required %zu", workspace_bytes, w.bytes);
      return -kErrWorkspace;
    }
#define B200_ATTN_ARGS q, k_pool, v_pool, block_table, ctx_lens, out, w, batch, num_q_heads, num_blocks, \
                       max_pages_per_seq, scale, split_tokens, ms, st
    if (head_dim == 128) {
      switch (num_kv_heads) {
        case 1: return launch_main<128, 1, 8, 4>(B200_ATTN_ARGS);
        case 2: return launch_main<128, 2, 6, 2>(B200_ATTN_ARGS);
        case 4:
          // measured on B200: few sequences (per-CTA fixed cost dominates) run best with three shallow CTAs per
          // SM, a full decode batch with two deeper ones
          if (batch <= 96) return launch_main<128, 4, 2, 3>(B200_ATTN_ARGS);
          return launch_main<128, 4, 3, 2>(B200_ATTN_ARGS);
        default: return launch_main<128, 8, 3, 1>(B200_ATTN_ARGS);
      }
    }
    switch (num_kv_heads) {
      case 1: return launch_main<64, 1, 8, 4>(B200_ATTN_ARGS);
      case 2: return launch_main<64, 2, 6, 4>(B200_ATTN_ARGS);
      case 4: return launch_main<64, 4, 6, 2>(B200_ATTN_ARGS);
      default: return launch_main<64, 8, 3, 2>(B200_ATTN_ARGS);
    }
#undef B200_ATTN_ARGS
  }
  int* err = static_cast<int*>(workspace);
  dim3 grid(num_q_heads, batch);
  if (dtype == 0)
    paged_attn_generic_kernel<__nv_bfloat16><<<grid, kGenWarps * 32, 0, st>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_pool),
        static_cast<const __nv_bfloat16*>(v_pool), block_table, ctx_lens,
        static_cast<__nv_bfloat16*>(out), err, num_q_heads, num_kv_heads, head_dim, page_size,
        num_blocks, max_pages_per_seq, scale);
  else
    paged_attn_generic_kernel<float><<<grid, kGenWarps * 32, 0, st>>>(
        static_cast<const float*>(q), static_cast<const float*>(k_pool),
        static_cast<const float*>(v_pool), block_table, ctx_lens, static_cast<float*>(out), err,
        num_q_heads, num_kv_heads, head_dim, page_size, num_blocks, max_pages_per_seq, scale);
  B200_CUDA(cudaGetLastError());
  return 0;
}

/* Prompt form: rows 2i and 2i+1 are two consecutive tokens of one sequence and share block_table row 2i. */
extern "C" int b200_paged_attn_decode_pairs(const void* q, const void* k_pool, const void* v_pool,
                                            const int32_t* block_table, const int32_t* ctx_lens, void* out,
                                            void* workspace, size_t workspace_bytes, int batch, int num_q_heads,
                                            int num_kv_heads, int head_dim, int page_size, int num_blocks,
                                            int max_pages_per_seq, float scale, int split_tokens, void* stream) {
  B200_REQUIRE(q && k_pool && v_pool && block_table && ctx_lens && out && workspace,
               "paged_attn_decode_pairs: null pointer");
  B200_REQUIRE(batch > 0 && num_q_heads > 0 && num_kv_heads > 0 && num_blocks > 0 && max_pages_per_seq > 0,
               "paged_attn_decode_pairs: non-positive dimension");
  B200_REQUIRE(num_q_heads % num_kv_heads == 0 && num_q_heads / num_kv_heads <= 8,
               "paged_attn_decode_pairs: %d query heads per kv head (at most 8: the second row uses the upper half "
               "of the MMA tile)", num_kv_heads ? num_q_heads / num_kv_heads : 0);
  B200_REQUIRE(page_size == kPage && split_tokens > 0 && split_tokens % kPage == 0,
               "paged_attn_decode_pairs: page_size %d must be %d and split_tokens %d a multiple of it", page_size, kPage,
               split_tokens);
  B200_REQUIRE((head_dim == 128 && num_kv_heads == 4) || (head_dim == 64 && num_kv_heads == 2),
               "paged_attn_decode_pairs: built for head_dim 128 with 4 kv heads and head_dim 64 with 2 kv heads, got "
               "%d / %d", head_dim, num_kv_heads);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(k_pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_pool) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(q) & 3) == 0,
               "paged_attn_decode_pairs: pools must be 16-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  const int ms = max_splits_of(max_pages_per_seq, page_size, split_tokens);
  B200_REQUIRE(ms <= 65535, "paged_attn_decode_pairs: grid too large");
  AttnWorkspace w = carve(workspace, batch, num_q_heads, head_dim, ms);
  if (workspace_bytes < w.bytes) {
    set_detail("paged_attn_decode_pairs: workspace %zu < required %zu", workspace_bytes, w.bytes);
    return -kErrWorkspace;
  }
  cudaStream_t st = as_stream(stream);
  if (head_dim == 128)
    return launch_main<128, 4, 3, 2, true>(q, k_pool, v_pool, block_table, ctx_lens, out, w, batch, num_q_heads,
                                           num_blocks, max_pages_per_seq, scale, split_tokens, ms, st);
  return launch_main<64, 2, 6, 4, true>(q, k_pool, v_pool, block_table, ctx_lens, out, w, batch, num_q_heads,
                                        num_blocks, max_pages_per_seq, scale, split_tokens, ms, st);
}

extern "C" int b200_kv_append(const void* k_new, const void* v_new, void* k_pool, void* v_pool,
                              const int32_t* block_table, const int32_t* positions,
                              void* status_word, int batch, int num_kv_heads, int head_dim,
                              int page_size, int num_blocks, int max_pages_per_seq, int dtype,
                              void* stream) {
  B200_REQUIRE(k_new && v_new && k_pool && v_pool && block_table && positions,
               "kv_append: null pointer");
  B200_REQUIRE(batch > 0 && num_kv_heads > 0 && head_dim > 0 && page_size > 0 && num_blocks > 0 &&
                   max_pages_per_seq > 0,
               "kv_append: non-positive dimension");
  B200_REQUIRE(dtype == 0 || dtype == 1, "kv_append: dtype %d is neither 0 (bf16) nor 1 (f32)", dtype);
  int rc = check_device(nullptr);
  if (rc) return rc;
  cudaStream_t st = as_stream(stream);
  const int threads = num_kv_heads * head_dim < 256 ? ((num_kv_heads * head_dim + 31) / 32) * 32 : 256;
  if (dtype == 0)
    kv_append_kernel<__nv_bfloat16><<<batch, threads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(k_new), static_cast<const __nv_bfloat16*>(v_new),
        static_cast<__nv_bfloat16*>(k_pool), static_cast<__nv_bfloat16*>(v_pool), block_table,
        positions, static_cast<int*>(status_word), num_kv_heads, head_dim, page_size, num_blocks,
        max_pages_per_seq);
  else
    kv_append_kernel<float><<<batch, threads, 0, st>>>(
        static_cast<const float*>(k_new), static_cast<const float*>(v_new),
        static_cast<float*>(k_pool), static_cast<float*>(v_pool), block_table, positions,
        static_cast<int*>(status_word), num_kv_heads, head_dim, page_size, num_blocks,
        max_pages_per_seq);
  B200_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------- allocation-free variant --
// Some hosts of this library cannot allocate device memory at the moment they
// need attention: a serving process whose memory pool was sized up front and is
// fully handed out, a plugin that is only lent buffers for its inputs and
// outputs, or code running while a CUDA graph is being captured (cudaMalloc is
// not allowed there).  For them the split partials live in a fixed array that is
// part of the library image.  Every GPU that loads the library carries these
// bytes until the process exits, so the size is kept modest.
constexpr size_t kStaticScratchBytes = B200_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

namespace b200 {
// Device address of the array above, per device.  In host code the array's name
// is only a handle for the runtime, not something a kernel can dereference; the
// usable address comes from cudaGetSymbolAddress with that device current.
static void* g_static_scratch_ptr[64] = {nullptr};
static std::mutex g_static_scratch_mu;

static int static_scratch_for_current_device(void** out) {
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_detail("paged_attn_decode_static: device index %d is outside the supported range", dev);
    return -kErrUnsupported;
  }
  std::lock_guard<std::mutex> lock(g_static_scratch_mu);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_attn_static_scratch)");
    g_static_scratch_ptr[dev] = p;
  }
  *out = g_static_scratch_ptr[dev];
  return 0;
}
}  // namespace b200

extern "C" int b200_paged_attn_decode_static(const void* q, const void* k_pool, const void* v_pool,
                                             const int32_t* block_table, const int32_t* ctx_lens,
                                             void* out, void* status_word, int batch,
                                             int num_q_heads, int num_kv_heads, int head_dim,
                                             int page_size, int num_blocks, int max_pages_per_seq,
                                             float scale, int split_tokens, void* stream) {
  B200_REQUIRE(q && k_pool && v_pool && block_table && ctx_lens && out,
               "paged_attn_decode_static: null pointer");
  B200_REQUIRE(batch > 0 && num_q_heads > 0 && num_kv_heads > 0 && num_blocks > 0 &&
                   max_pages_per_seq > 0 && split_tokens > 0,
               "paged_attn_decode_static: non-positive dimension");
  B200_REQUIRE(num_q_heads % num_kv_heads == 0 && num_q_heads / num_kv_heads <= 16,
               "paged_attn_decode_static: need at most 16 q heads per kv head (%d / %d)", num_q_heads,
               num_kv_heads);
  B200_REQUIRE(page_size == kPage && (head_dim == 64 || head_dim == 128) &&
                   (num_kv_heads == 1 || num_kv_heads == 2 || num_kv_heads == 4 || num_kv_heads == 8),
               "paged_attn_decode_static: only the split-K kernel is offered here (bf16, page 16, head_dim "
               "64 or 128, 1/2/4/8 kv heads)");
  B200_REQUIRE(split_tokens % kPage == 0, "paged_attn_decode_static: split_tokens %d not a multiple of %d",
               split_tokens, kPage);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(k_pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_pool) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(q) & 3) == 0,
               "paged_attn_decode_static: pools must be 16-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  const int ms = max_splits_of(max_pages_per_seq, page_size, split_tokens);
  B200_REQUIRE(ms <= 65535, "paged_attn_decode_static: grid too large");
  // Lay the partials out in the static array exactly as carve() does in a caller workspace,
  // minus the status block: the status word here is the caller's.
  const size_t ml_bytes = (static_cast<size_t>(batch) * num_q_heads * ms * sizeof(float2) + 255) & ~size_t(255);
  const size_t o_bytes = static_cast<size_t>(batch) * num_q_heads * ms * head_dim * sizeof(float);
  if (ml_bytes + o_bytes > kStaticScratchBytes) {
    set_detail("paged_attn_decode_static: batch %d x %d heads x %d splits needs %zu bytes of split partials; the "
               "built-in scratch holds %zu. Use fewer splits (larger split_tokens), a smaller batch, or "
               "b200_paged_attn_decode with a workspace of your own.",
               batch, num_q_heads, ms, ml_bytes + o_bytes, kStaticScratchBytes);
    return -kErrWorkspace;
  }
  void* scratch = nullptr;
  rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;
  AttnWorkspace w;
  w.err = static_cast<int*>(status_word);
  w.ml = reinterpret_cast<float2*>(scratch);
  w.o = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + ml_bytes);
  w.bytes = ml_bytes + o_bytes;
  cudaStream_t st = as_stream(stream);
#define B200_ATTN_ARGS q, k_pool, v_pool, block_table, ctx_lens, out, w, batch, num_q_heads, num_blocks, \
                       max_pages_per_seq, scale, split_tokens, ms, st
  if (head_dim == 128) {
    switch (num_kv_heads) {
      case 1: return launch_main<128, 1, 8, 4>(B200_ATTN_ARGS);
      case 2: return launch_main<128, 2, 6, 2>(B200_ATTN_ARGS);
      case 4: return launch_main<128, 4, 3, 2>(B200_ATTN_ARGS);
      default: return launch_main<128, 8, 3, 1>(B200_ATTN_ARGS);
    }
  }
  switch (num_kv_heads) {
    case 1: return launch_main<64, 1, 8, 4>(B200_ATTN_ARGS);
    case 2: return launch_main<64, 2, 6, 4>(B200_ATTN_ARGS);
    case 4: return launch_main<64, 4, 6, 2>(B200_ATTN_ARGS);
    default: return launch_main<64, 8, 3, 2>(B200_ATTN_ARGS);
  }
#undef B200_ATTN_ARGS
}
