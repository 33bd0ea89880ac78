// Tiled causal attention over KV pages for a chunk of prompt tokens (sm_100a).
//
// The reference runs a prompt (or the uncached suffix of one) through the model with a dense cache:
// cached prefix pages are first gathered into a [1, H, S, D] tensor
// (src/inference_server/kv_cache/hf_format.py:21-45), then the suffix attends to prefix + itself
// under a causal mask inside the model forward (src/inference_server/backends/torch_backend.py:107-147,
// chunked: src/inference_server/scheduler.py:312-353).  Here a chunk of R consecutive prompt tokens of
// one sequence (positions first_pos .. first_pos + R - 1, whose K/V are already in their page slots)
// attends straight to the sequence's pages, cached prefix pages included, flash-attention style:
//
//   grid  = (query tiles, kv heads).  A CTA owns 128 rows of the score matrix: 128 / G consecutive
//           prompt positions x the G query heads that share the kv head, so a K/V page fetched once
//           serves 128 rows (the decode kernel's row-per-token form serves 8 or 16).
//   load  = one producer warp walks the block table and brings page after page of its kv head into a
//           ring of one-page stages: TMA boxes of 16 tokens x 128 B, 128-byte swizzle, mbarrier
//           hand-over.
//   math  = 8 consumer warps, one m16 tile (16 score rows) each.  Four warps with two tiles each share
//           more K/V fragments per warp but need 255 registers and leave a scheduler with one warp:
//           measured 25 % tensor-pipe activity, stalled on fixed-latency dependencies; eight lighter
//           warps hide them better.  S = Q K^T by mma.sync m16n8k16, causal mask by position (row of position p sees tokens
//           0..p), online softmax in fp32 in the log2 domain, O += P V.  No split over the context
//           and no second pass: a row's whole context is inside one CTA.
//   out   = normalised bf16 rows written from registers.
// Heavy tiles (late positions, long context) are issued first.

#include <stdlib.h>

#include "common.cuh"
#include "host.h"

namespace b200 {

constexpr int kPfPage = 16;
constexpr int kPfRows = 128;        // score-matrix rows per CTA
constexpr int kPfMt = 1;            // m16 tiles per consumer warp (they share every K and V fragment)
constexpr int kPfWarps = kPfRows / (16 * kPfMt);  // consumer warps
constexpr int kPfStages = 8;

template <int D>
struct PrefillCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kBoxBytes = kPfPage * 128;              // 16 tokens x 128 B
  static constexpr int kStageBytes = 2 * kHalves * kBoxBytes;  // K halves then V halves
  static constexpr int kRingBytes = kPfStages * kStageBytes;
  static constexpr int kSmemBytes = kRingBytes + 1024 + 16 * kPfStages;
  static constexpr int kThreads = (kPfWarps + 1) * 32;
};

// G: query heads per kv head (4, 8 or 16).
template <int D, int G>
__global__ void __launch_bounds__((kPfWarps + 1) * 32, 1)
paged_attn_prefill_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                          const __nv_bfloat16* __restrict__ q, const int* __restrict__ table_row,
                          __nv_bfloat16* __restrict__ out, int* __restrict__ err, int num_tokens, int first_pos,
                          int num_q_heads, int num_kv_heads, int num_blocks, int max_pages, float scale_log2) {
#ifdef B200_DEVICE_OK
  using Cfg = PrefillCfg<D>;
  constexpr int QT = kPfRows / G;  // prompt positions per CTA
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = ring + Cfg::kRingBytes;  // full[kPfStages], empty[kPfStages]

  const int tiles = (num_tokens + QT - 1) / QT;
  const int tile = tiles - 1 - static_cast<int>(blockIdx.x);  // longest contexts first
  const int kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i0 = tile * QT;                                   // first chunk index of this tile
  const int i_last = min(i0 + QT, num_tokens) - 1;            // last real chunk index
  int l_max = first_pos + i_last + 1;                         // tokens the last row sees
  const int l_min = first_pos + i0 + 1;                       // tokens the first row sees
  if (l_max > max_pages * kPfPage || first_pos < 0) {
    if (threadIdx.x == 0) set_error(err, kErrDevBadCtxLen);
    l_max = min(max(l_max, 1), max_pages * kPfPage);
  }
  const int npages = (l_max + kPfPage - 1) / kPfPage;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPfStages; ++s) {
      mbar_init(bars + 8 * s, 1);
      mbar_init(bars + 8 * (kPfStages + s), kPfWarps);
    }
    fence_mbar_init();
    fence_proxy_async();
  }
  __syncthreads();

  if (warp == kPfWarps) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
    }
    const int lkv = lane / Cfg::kHalves, lh = lane % Cfg::kHalves;  // lane -> (K or V, column half)
    const bool issuer = lane < 2 * Cfg::kHalves;
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
      const int slot = i % kPfStages;
      const uint32_t phase = (i / kPfStages) & 1;
      if (!mbar_wait(bars + 8 * (kPfStages + slot), phase ^ 1, err)) break;
      if (lane == 0) mbar_arrive_expect_tx(bars + 8 * slot, Cfg::kStageBytes);
      __syncwarp();
      if (issuer) {
        const uint32_t dst = ring + slot * Cfg::kStageBytes + (lkv * Cfg::kHalves + lh) * Cfg::kBoxBytes;
        tma_load_2d(dst, lkv ? &v_map : &k_map, bars + 8 * slot, lh * 64, (id * num_kv_heads + kvh) * kPfPage);
      }
    }
    return;
  }

  // --------------------------------------------------------------- consumers --
  const int gq = lane >> 2, tq = lane & 3;
  // this thread's four score rows: m16 tile mt, fragment rows gq and gq + 8
  int len[kPfMt][2];        // tokens the row sees (its position + 1); rows past the chunk copy the tile's first row
  bool real[kPfMt][2];
  const __nv_bfloat16* qrow[kPfMt][2];
  __nv_bfloat16* orow[kPfMt][2];
#pragma unroll
  for (int mt = 0; mt < kPfMt; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = warp * (16 * kPfMt) + mt * 16 + h * 8 + gq;  // row inside the CTA
      const int pos_i = i0 + r / G, head = kvh * G + r % G;
      real[mt][h] = pos_i < num_tokens;
      const int ii = real[mt][h] ? pos_i : i0;
      len[mt][h] = first_pos + ii + 1;
      qrow[mt][h] = q + (static_cast<size_t>(ii) * num_q_heads + head) * D;
      orow[mt][h] = out + (static_cast<size_t>(ii) * num_q_heads + head) * D;
    }

  uint32_t qa[kPfMt][D / 16][4];
#pragma unroll
  for (int mt = 0; mt < kPfMt; ++mt)
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int d0 = ks * 16 + 2 * tq;
      const uint32_t* r0 = reinterpret_cast<const uint32_t*>(qrow[mt][0] + d0);
      const uint32_t* r1 = reinterpret_cast<const uint32_t*>(qrow[mt][1] + d0);
      qa[mt][ks][0] = __ldg(r0);
      qa[mt][ks][1] = __ldg(r1);
      qa[mt][ks][2] = __ldg(r0 + 4);
      qa[mt][ks][3] = __ldg(r1 + 4);
    }

  float o[kPfMt][D / 8][4];
#pragma unroll
  for (int mt = 0; mt < kPfMt; ++mt)
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[mt][n][0] = o[mt][n][1] = o[mt][n][2] = o[mt][n][3] = 0.f;
  float mrun[kPfMt][2], lrun[kPfMt][2];
#pragma unroll
  for (int mt = 0; mt < kPfMt; ++mt) {
    mrun[mt][0] = mrun[mt][1] = -INFINITY;
    lrun[mt][0] = lrun[mt][1] = 0.f;
  }

  const int lj = lane >> 3, lr = lane & 7;
  const int k_tok = (lj >> 1) * 8 + lr, k_sub = lj & 1;
  const int v_tok = (lj & 1) * 8 + lr, v_sub = lj >> 1;

  bool alive = true;
  for (int i = 0; i < npages && alive; ++i) {
    const int slot = i % kPfStages;
    const uint32_t phase = (i / kPfStages) & 1;
    alive = mbar_wait(bars + 8 * slot, phase, err);
    if (alive) {
      const uint32_t kbase = ring + slot * Cfg::kStageBytes;
      const uint32_t vbase = kbase + Cfg::kHalves * Cfg::kBoxBytes;

      float s0[kPfMt][4], s1[kPfMt][4];
#pragma unroll
      for (int mt = 0; mt < kPfMt; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s0[mt][e] = s1[mt][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int cidx = ks * 2 + k_sub;
        uint32_t b00, b01, b10, b11;
        ldmatrix_x4(kbase + (cidx >> 3) * Cfg::kBoxBytes + swz128(k_tok, cidx & 7), b00, b01, b10, b11);
#pragma unroll
        for (int mt = 0; mt < kPfMt; ++mt) {
          mma_bf16_16816(s0[mt], qa[mt][ks], b00, b01);
          mma_bf16_16816(s1[mt], qa[mt][ks], b10, b11);
        }
      }

      const int tok0 = i * kPfPage + 2 * tq;  // token of s0[.][0]; s0[.][1] is +1, s1 is +8
      const bool edge = i * kPfPage + kPfPage > l_min;  // some row of the CTA ends inside or before this page
      uint32_t pa[kPfMt][4];
      float alpha[kPfMt][2];
#pragma unroll
      for (int mt = 0; mt < kPfMt; ++mt) {
        if (edge) {
          const int la = len[mt][0], lb = len[mt][1];
          if (tok0 >= la) s0[mt][0] = -INFINITY;
          if (tok0 + 1 >= la) s0[mt][1] = -INFINITY;
          if (tok0 + 8 >= la) s1[mt][0] = -INFINITY;
          if (tok0 + 9 >= la) s1[mt][1] = -INFINITY;
          if (tok0 >= lb) s0[mt][2] = -INFINITY;
          if (tok0 + 1 >= lb) s0[mt][3] = -INFINITY;
          if (tok0 + 8 >= lb) s1[mt][2] = -INFINITY;
          if (tok0 + 9 >= lb) s1[mt][3] = -INFINITY;
        }
        float p[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float mx = fmaxf(fmaxf(s0[mt][2 * h], s0[mt][2 * h + 1]), fmaxf(s1[mt][2 * h], s1[mt][2 * h + 1]));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          // every row sees token 0, so after the first page its running maximum is finite; a page that lies
          // wholly behind a row's end leaves the row untouched (all its exponentials are 0)
          const float mnew = fmaxf(mrun[mt][h], mx * scale_log2);
          const float mref = mnew == -INFINITY ? 0.f : mnew;
          alpha[mt][h] = exp2f(mrun[mt][h] - mref);
          mrun[mt][h] = mnew;
          p[h][0] = exp2f(s0[mt][2 * h] * scale_log2 - mref);
          p[h][1] = exp2f(s0[mt][2 * h + 1] * scale_log2 - mref);
          p[h][2] = exp2f(s1[mt][2 * h] * scale_log2 - mref);
          p[h][3] = exp2f(s1[mt][2 * h + 1] * scale_log2 - mref);
          lrun[mt][h] = lrun[mt][h] * alpha[mt][h] + (p[h][0] + p[h][1]) + (p[h][2] + p[h][3]);
        }
        pa[mt][0] = pack_bf16x2(p[0][0], p[0][1]);
        pa[mt][1] = pack_bf16x2(p[1][0], p[1][1]);
        pa[mt][2] = pack_bf16x2(p[0][2], p[0][3]);
        pa[mt][3] = pack_bf16x2(p[1][2], p[1][3]);
      }
      bool resc = false;
#pragma unroll
      for (int mt = 0; mt < kPfMt; ++mt) resc = resc || alpha[mt][0] != 1.f || alpha[mt][1] != 1.f;
      const bool rescale = __any_sync(0xffffffffu, resc);
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
        if (rescale) {
#pragma unroll
          for (int mt = 0; mt < kPfMt; ++mt) {
            o[mt][2 * np][0] *= alpha[mt][0];
            o[mt][2 * np][1] *= alpha[mt][0];
            o[mt][2 * np + 1][0] *= alpha[mt][0];
            o[mt][2 * np + 1][1] *= alpha[mt][0];
            o[mt][2 * np][2] *= alpha[mt][1];
            o[mt][2 * np][3] *= alpha[mt][1];
            o[mt][2 * np + 1][2] *= alpha[mt][1];
            o[mt][2 * np + 1][3] *= alpha[mt][1];
          }
        }
        const int cidx = np * 2 + v_sub;
        uint32_t v0, v1, v2, v3;
        ldmatrix_x4_trans(vbase + (cidx >> 3) * Cfg::kBoxBytes + swz128(v_tok, cidx & 7), v0, v1, v2, v3);
#pragma unroll
        for (int mt = 0; mt < kPfMt; ++mt) {
          mma_bf16_16816(o[mt][2 * np], pa[mt], v0, v1);
          mma_bf16_16816(o[mt][2 * np + 1], pa[mt], v2, v3);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bars + 8 * (kPfStages + slot));
  }
  if (!alive) return;

#pragma unroll
  for (int mt = 0; mt < kPfMt; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float l = lrun[mt][h];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const float inv = 1.f / l;
      if (real[mt][h]) {
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
          *reinterpret_cast<uint32_t*>(orow[mt][h] + n * 8 + 2 * tq) =
              pack_bf16x2(o[mt][n][2 * h] * inv, o[mt][n][2 * h + 1] * inv);
      }
    }
#endif
}

template <int D, int G>
static int launch_prefill(const void* q, const void* k_pool, const void* v_pool, const int* table_row, void* out,
                          int* err, int num_tokens, int first_pos, int hq, int hkv, int num_blocks, int max_pages,
                          float scale, cudaStream_t st) {
  using Cfg = PrefillCfg<D>;
  CUtensorMap kmap, vmap;
  const uint64_t rows = static_cast<uint64_t>(num_blocks) * hkv * kPfPage;
  int rc = get_tensor_map_2d(k_pool, rows, D, 2, kPfPage, 64, &kmap);
  if (rc) return rc;
  rc = get_tensor_map_2d(v_pool, rows, D, 2, kPfPage, 64, &vmap);
  if (rc) return rc;
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&paged_attn_prefill_kernel<D, G>), Cfg::kSmemBytes);
  if (rc) return rc;
  constexpr int QT = kPfRows / G;
  dim3 grid((num_tokens + QT - 1) / QT, hkv);
  paged_attn_prefill_kernel<D, G><<<grid, Cfg::kThreads, Cfg::kSmemBytes, st>>>(
      kmap, vmap, static_cast<const __nv_bfloat16*>(q), table_row, static_cast<__nv_bfloat16*>(out), err, num_tokens,
      first_pos, hq, hkv, num_blocks, max_pages, scale * 1.4426950408889634f);
  B200_CUDA(cudaGetLastError());
  return 0;
}

// paged_prefill_tc.cu
int launch_prefill_tc(const void* q, const void* k_pool, const void* v_pool, const int* table_row, void* out, int* err,
                      int num_tokens, int first_pos, int hq, int hkv, int num_blocks, float scale, cudaStream_t st);

// The tcgen05 kernel serves head_dim 128 unless the environment variable B200_PREFILL_MMA_SYNC is set to a
// non-zero value (read once), which keeps every shape on the mma.sync kernel of this file.
static bool prefill_tc_enabled() {
  static const bool enabled = [] {
    const char* v = getenv("B200_PREFILL_MMA_SYNC");
    return !(v && v[0] != '\0' && v[0] != '0');
  }();
  return enabled;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_paged_attn_prefill(const void* q, const void* k_pool, const void* v_pool,
                                       const int32_t* block_table_row, void* out, void* status_word, int num_tokens,
                                       int first_position, int num_q_heads, int num_kv_heads, int head_dim,
                                       int page_size, int num_blocks, int max_pages_per_seq, float scale,
                                       void* stream) {
  B200_REQUIRE(q && k_pool && v_pool && block_table_row && out, "paged_attn_prefill: null pointer");
  B200_REQUIRE(num_tokens > 0 && first_position >= 0 && num_q_heads > 0 && num_kv_heads > 0 && num_blocks > 0 &&
                   max_pages_per_seq > 0,
               "paged_attn_prefill: non-positive dimension");
  B200_REQUIRE(page_size == kPfPage, "paged_attn_prefill: page_size %d must be %d", page_size, kPfPage);
  B200_REQUIRE(num_q_heads % num_kv_heads == 0, "paged_attn_prefill: q heads %d not a multiple of kv heads %d",
               num_q_heads, num_kv_heads);
  const int group = num_q_heads / num_kv_heads;
  B200_REQUIRE((head_dim == 128 && (group == 8 || group == 16)) || (head_dim == 64 && group == 4),
               "paged_attn_prefill: built for head_dim 128 with 8 or 16 query heads per kv head and head_dim 64 with "
               "4, got %d / %d", head_dim, group);
  B200_REQUIRE(first_position + num_tokens <= max_pages_per_seq * kPfPage,
               "paged_attn_prefill: positions up to %d do not fit %d pages", first_position + num_tokens,
               max_pages_per_seq);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(k_pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(v_pool) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(q) & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0,
               "paged_attn_prefill: pools must be 16-byte aligned, q and out 4-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  cudaStream_t st = as_stream(stream);
  int* err = static_cast<int*>(status_word);
#define B200_PF_ARGS q, k_pool, v_pool, block_table_row, out, err, num_tokens, first_position, num_q_heads, \
                     num_kv_heads, num_blocks, max_pages_per_seq, scale, st
  if (head_dim == 128 && prefill_tc_enabled() &&
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15) == 0)
    return launch_prefill_tc(q, k_pool, v_pool, block_table_row, out, err, num_tokens, first_position, num_q_heads,
                             num_kv_heads, num_blocks, scale, st);
  if (head_dim == 128 && group == 8) return launch_prefill<128, 8>(B200_PF_ARGS);
  if (head_dim == 128) return launch_prefill<128, 16>(B200_PF_ARGS);
  return launch_prefill<64, 4>(B200_PF_ARGS);
#undef B200_PF_ARGS
}
