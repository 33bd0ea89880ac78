// Dense bf16 projections of the decode step on the tensor cores (tcgen05 / TMEM), sm_100a.
//
// Replaces the linear layers that the reference's model forward runs as library GEMMs
// (src/inference_server/backends/torch_backend.py:314-320 -> transformers Qwen3MoeAttention q/k/v/o
// projections, the router's gate projection and lm_head), and the argmax over the vocabulary that
// follows lm_head (torch_backend.py:321):
//     Y[m, n] = sum_k X[m, k] * W[n, k]        X [M, K] bf16, W [N, K] bf16, fp32 accumulation
//
// A decode step has few rows (M = the batch, up to a few hundred) and large weights, so the kernel
// is laid out around the weight stream: a 128-row tile of W is the M side of tcgen05.mma (A operand,
// K-major, straight from the checkpoint layout) and the step's rows are the N side (B operand, up to
// 256 rows per MMA).  The accumulator in TMEM therefore holds Y transposed: lane = output feature,
// column = row of X.
//
//   warp 0      TMA producer: per 64-wide K block one or two W boxes (128 rows x 128 B) and one X
//               box (32..256 rows x 128 B) into an mbarrier ring, 128-byte swizzle.
//   warp 1      MMA issuer: one thread issues 4 x tcgen05.mma (M128, N = X box rows, K16,
//               kind::f16 on bf16) per K block and W tile; commits to the stage-empty barrier and,
//               after the last K block, to the accumulator-full barrier.
//   warps 2-9   epilogue: tcgen05.ld of the accumulator, 32 columns (rows of X) at a time; warps 2-5
//               and 6-9 each cover the four TMEM lane quarters and share the columns between them.
//
// A work item is (128-row weight tile, tile of 32..256 rows of X, slice of K).  Three things keep a small
// problem busy on 148 SMs; the host picks among them with a small cost model (bytes each CTA pulls, waves,
// cost of the partial exchange):
//   row tiles   the step's rows are cut into tiles narrower than the batch: more items, each pulling less
//               of X; the weight tile is then read once per row tile, from L2 after the first.
//   split K     qkv / o / router have only 1..72 weight tiles.  K is split over the CTAs of a
//               thread-block cluster (2, 4 or 8), which the hardware schedules together.  Every CTA
//               writes its fp32 partial tile to a caller workspace, grouped by the CTA that will
//               finish those rows; after one cluster barrier (release / acquire at cluster scope)
//               CTA r sums, in rank order, the partials of all CTAs for its share of the rows and
//               writes bf16.  The partials live a few microseconds and stay in L2.  Deterministic:
//               no atomics.  (Distributed shared memory was measured for this exchange and is several
//               times slower: about 12 bytes per clock per SM against the 128 KiB each CTA must move.)
//               The split is chosen so that all clusters of the launch are resident at once
//               (cudaOccupancyMaxActiveClusters).
//   two tiles   lm_head has 1187 weight tiles and needs no split; there a CTA takes two adjacent
//               128-row tiles of W against one X box (two accumulators), which halves how often X
//               is pulled from L2, and walks its share of the vocabulary persistently.
//
// Epilogues: bf16 store, or (lm_head) a running arg-max: every epilogue thread owns one feature of
// the current weight tile and keeps, for each of its 128 rows of X, the largest logit it has seen over
// all the tiles of the CTA as one integer key in a register; the warp-wide maximum is taken once, after
// the last tile.  The [M, vocab] logits are never written; a small second kernel folds the per-warp
// candidates (largest value, ties to the lower token id).

#include <mutex>

#include <stdlib.h>

#include "common.cuh"
#include "host.h"

namespace b200 {

constexpr int kDenseBlockK = 64;                  // bf16 elements per K block: 128 bytes
constexpr int kDenseWBytes = 128 * 128;           // one W tile of a stage
constexpr int kDenseXBytesMax = 256 * 128;        // largest X box of a stage
constexpr int kDenseThreads = 10 * 32;           // TMA warp, MMA warp, 8 epilogue warps
constexpr int kDenseMaxRows = 256;                // rows of X per MMA (its N)

enum : int { kEpiStore = 0, kEpiArgmax = 1, kEpiQkvRope = 2 };
constexpr int kQkvStageBytes = kDenseMaxRows * 128 * 2;  // kEpiQkvRope: one head of up to 256 rows, bf16

template <int A_TILES, int EPI = kEpiStore>
struct DenseCfg {
  // the q/k/v epilogue keeps a bf16 copy of one head's tile beside the ring and gives a stage for it
  static constexpr int kStages = (A_TILES == 1 && EPI != kEpiQkvRope) ? 4 : 3;
  static constexpr int kStageBytes = A_TILES * kDenseWBytes + kDenseXBytesMax;
  static constexpr int kRingBytes = kStages * kStageBytes;  // 192 KiB, or 144 KiB + 64 KiB of head tile
  static constexpr int kExtraBytes = EPI == kEpiQkvRope ? kQkvStageBytes : 0;
  static constexpr int kSmemBytes = kRingBytes + kExtraBytes + 1024 /* alignment */ + 256 /* barriers, tmem base */;
};

struct DenseParams {
  __nv_bfloat16* y;   // kEpiStore: [M, N]
  float* part_val;    // kEpiArgmax: [grid * 4, 256] candidates per TMEM lane quarter
  int* part_idx;
  float* exchange;    // kEpiStore, split K: [tile][finishing CTA][source CTA][rows_per][128] fp32
  // kEpiQkvRope: the q/k/v projection of heads of 128 with per-head RMSNorm, RoPE and the page write in its
  // epilogue (what b200_qk_norm_rope_append does after a plain projection)
  const __nv_bfloat16* q_norm_w;
  const __nv_bfloat16* k_norm_w;
  const __nv_bfloat16* cos_t;
  const __nv_bfloat16* sin_t;
  const int* positions;
  const int* block_table;
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_pool;
  __nv_bfloat16* v_pool;
  float eps;
  int hq, hkv, page, num_blocks, max_pages, max_pos;
  int* err;
  int M, N, K;
  int m_tiles;        // ceil(M / xbox)
  int n_tiles;        // ceil(N / (128 * A_TILES))
  int ksplit;         // CTAs of a cluster that share one tile (1 = no cluster)
  int xbox;           // rows of X per work item = rows of the X box = N of the MMA: a multiple of 32 up to 256
                      // (a power of two wherever K is split)
};

// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(uint32_t m, uint32_t n) {
  return (1u << 4)            // accumulator f32
         | (1u << 7)          // A bf16
         | (1u << 10)         // B bf16
         | ((n >> 3) << 17)   // N
         | ((m >> 4) << 24);  // M
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---- thread-block cluster helpers (split K) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Every thread of every CTA of the cluster takes part; release/acquire orders the shared-memory
// writes before it against the remote reads after it.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Order-preserving map of a float onto an unsigned integer (and back): a < b  <=>  key(a) < key(b).
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return u ^ ((u >> 31) ? 0xffffffffu : 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  return __uint_as_float(k ^ ((k >> 31) ? 0x80000000u : 0xffffffffu));
}

template <int A_TILES, int EPI>
__global__ void __launch_bounds__(kDenseThreads, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                  const DenseParams p) {
#ifdef B200_DEVICE_OK
  using Cfg = DenseCfg<A_TILES, EPI>;
  constexpr int kStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
  const uint32_t bars = ring + Cfg::kRingBytes + Cfg::kExtraBytes;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kStages;
  const uint32_t bar_tfull = bars + 16 * kStages, bar_tempty = bar_tfull + 16;
  uint32_t* tmem_base_sm = reinterpret_cast<uint32_t*>(ring_ptr + Cfg::kRingBytes + Cfg::kExtraBytes + 16 * kStages + 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // accumulator buffers: one W tile -> two buffers of 256 columns that alternate between work items;
  // two W tiles -> both halves of TMEM belong to one item
  constexpr int kBufs = A_TILES == 1 ? 2 : 1;

  if (threadIdx.x == 32) {  // warm the descriptor cache while the barriers and TMEM are being set up
    tma_prefetch_desc(&w_map);
    tma_prefetch_desc(&x_map);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, 8);
    }
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_base_sm), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_sm;
  // Everything above is this CTA's own set-up; X (and the buffers the epilogues write) belong to the kernels
  // before this one.
  grid_dep_wait();
  grid_dep_launch();

  const int ks = p.ksplit;
  const int kb_per = p.K / kDenseBlockK / ks;  // K blocks of one work item
  const int total = p.n_tiles * p.m_tiles * ks;
  const uint32_t stage_tx = A_TILES * kDenseWBytes + static_cast<uint32_t>(p.xbox) * 128u;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA ------
    if (lane == 0) {
      uint32_t it = 0;
      bool alive = true;
      for (int w = blockIdx.x; w < total && alive; w += gridDim.x) {
        const int tile = w / ks, kidx = w - tile * ks;
        const int nt = tile / p.m_tiles, mt = tile - nt * p.m_tiles;
        for (int kb = 0; kb < kb_per; ++kb, ++it) {
          const uint32_t slot = it % kStages, phase = (it / kStages) & 1;
          alive = mbar_wait(bar_empty + 8 * slot, phase ^ 1, p.err);
          if (!alive) break;
          const uint32_t sw = ring + slot * Cfg::kStageBytes, sx = sw + A_TILES * kDenseWBytes;
          const int kx = (kidx * kb_per + kb) * kDenseBlockK;
          mbar_arrive_expect_tx(bar_full + 8 * slot, stage_tx);
#pragma unroll
          for (int a = 0; a < A_TILES; ++a)
            tma_load_2d(sw + a * kDenseWBytes, &w_map, bar_full + 8 * slot, kx, (nt * A_TILES + a) * 128);
          tma_load_2d(sx, &x_map, bar_full + 8 * slot, kx, mt * p.xbox);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA ------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(128, static_cast<uint32_t>(p.xbox));
      uint32_t it = 0, item = 0;
      bool alive = true;
      for (int w = blockIdx.x; w < total && alive; w += gridDim.x, ++item) {
        const uint32_t buf = item % kBufs, aphase = (item / kBufs) & 1;
        alive = mbar_wait(bar_tempty + 8 * buf, aphase ^ 1, p.err);
        if (!alive) break;
        tc_fence_after();
        for (int kb = 0; kb < kb_per; ++kb, ++it) {
          const uint32_t slot = it % kStages, phase = (it / kStages) & 1;
          alive = mbar_wait(bar_full + 8 * slot, phase, p.err);
          if (!alive) break;
          tc_fence_after();
          const uint32_t sw = ring + slot * Cfg::kStageBytes, sx = sw + A_TILES * kDenseWBytes;
          const uint64_t b_desc = umma_desc_k128(sx);
#pragma unroll
          for (int a = 0; a < A_TILES; ++a) {
            const uint64_t a_desc = umma_desc_k128(sw + a * kDenseWBytes);
            const uint32_t d = tmem_base + (A_TILES == 1 ? buf : static_cast<uint32_t>(a)) * kDenseMaxRows;
#pragma unroll
            for (int k = 0; k < kDenseBlockK / 16; ++k)
              tc_mma_bf16(d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(bar_empty + 8 * slot);
        }
        if (alive) tc_commit(bar_tfull + 8 * buf);
      }
    }
  } else if (EPI == kEpiStore && ks > 1) {
    // ------------------------------------- epilogue, split K: wait only ------
    // one work item per CTA; the accumulator is read after the cluster barrier below
    if (static_cast<int>(blockIdx.x) < total) mbar_wait(bar_tfull, 0, p.err);
    tc_fence_after();
  } else {
    // ------------------------------------------------------- epilogue ------
    const int quarter = warp & 3;        // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;    // warps 2-5: 0, warps 6-9: 1
    const int t = quarter * 32 + lane;   // feature inside a 128-row W tile
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int chunks = p.xbox / 32;
    // arg-max state: best[j] is the largest key this thread has seen for row half * 128 + j of X.  A key is
    // the order-preserving integer image of the fp32 logit with its five lowest bits replaced by 31 - (ordinal
    // of the weight tile within this CTA): an integer max keeps the largest logit (to 2^-18 relative, finer than
    // the accumulation order resolves) and, among equal ones, the earliest tile, i.e. the lowest token id.
    uint32_t best[EPI == kEpiArgmax ? 128 : 1];
#pragma unroll
    for (int j = 0; j < (EPI == kEpiArgmax ? 128 : 1); ++j) best[j] = 0u;
    uint32_t item = 0;
    bool alive = true;
    for (int w = blockIdx.x; w < total && alive; w += gridDim.x, ++item) {
      const int tile = w / ks;
      const int nt = tile / p.m_tiles, mt = tile - nt * p.m_tiles;
      const uint32_t buf = item % kBufs, aphase = (item / kBufs) & 1;
      const int m0 = mt * p.xbox;
      // kEpiQkvRope: position and page of the rows this warp will finish (lane i: row (warp - 2) + 8 i of the
      // tile), fetched while the MMAs of the item are still running; -1 = not a row, or reported as bad
      int row_pos = -1, row_page = -1;
      if (EPI == kEpiQkvRope) {
        const int r = (warp - 2) + 8 * lane, m = m0 + r;
        if (r < p.xbox && m < p.M) {
          const int ps = p.positions[m];
          if (ps < 0 || ps >= p.max_pos || ps >= p.max_pages * p.page) {
            set_error(p.err, kErrDevBadCtxLen);
          } else {
            row_pos = ps;
            if (nt >= p.hq) {  // k and v heads go to the page of that position
              const int id = p.block_table[static_cast<size_t>(m) * p.max_pages + ps / p.page];
              if (id < 0 || id >= p.num_blocks) set_error(p.err, kErrDevBadBlockId);
              else row_page = id;
            }
          }
        }
      }
      alive = mbar_wait(bar_tfull + 8 * buf, aphase, p.err);
      if (!alive) break;
      tc_fence_after();
#pragma unroll
      for (int a = 0; a < A_TILES; ++a) {
        const int n = (nt * A_TILES + a) * 128 + t;
        const uint32_t t0 = lane_addr + (A_TILES == 1 ? buf : static_cast<uint32_t>(a)) * kDenseMaxRows;
        if (EPI == kEpiQkvRope) {
          // the tile is one head (128 features) of up to 256 rows: a bf16 copy goes to shared memory as
          // [row][feature] - the projection's output is bf16 in the model, so this rounding is the model's
          __nv_bfloat16* head = reinterpret_cast<__nv_bfloat16*>(ring_ptr + Cfg::kRingBytes);
          for (int c = half; c < chunks; c += 2) {
            uint32_t v[32];
            tmem_ld32(t0 + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) head[(c * 32 + i) * 128 + t] = __float2bfloat16(__uint_as_float(v[i]));
          }
        } else if (EPI == kEpiStore) {
          for (int c = half; c < chunks; c += 2) {
            uint32_t v[32];
            tmem_ld32(t0 + c * 32, v);
            tmem_ld_wait();
            if (n < p.N) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int m = m0 + c * 32 + i;
                if (m < p.M) p.y[static_cast<size_t>(m) * p.N + n] = __float2bfloat16(__uint_as_float(v[i]));
              }
            }
          }
        } else {
          const uint32_t tag = 31u - (item * A_TILES + a);  // at most 32 weight tiles per CTA (checked on the host)
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (half * 4 + c < chunks) {
              uint32_t v[32];
              tmem_ld32(t0 + (half * 4 + c) * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const uint32_t key = n < p.N ? ((float_key(__uint_as_float(v[i])) & ~31u) | tag) : 0u;
                best[EPI == kEpiArgmax ? c * 32 + i : 0] = max(best[EPI == kEpiArgmax ? c * 32 + i : 0], key);
              }
            }
          }
        }
      }
      // everything this thread needs from the accumulator is in registers (or shared memory)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
      if (EPI == kEpiQkvRope) {
        // ---- per row of X: RMSNorm over the head (q and k), RoPE (rotate-half), then q to its output row
        // and k / v into their page slot; warp e takes rows e, e + 8, ...; lane l holds d = l + 32 j.  Position
        // and page of every row were fetched before the accumulator was awaited (lane i: the warp's i-th row), and
        // the rows go four at a time so that their cos/sin loads are in flight together: done one row after the
        // other, the dependent loads of 16-32 rows per warp cost more than the separate kernel they replace.
        asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight epilogue warps: the head tile is complete
        const __nv_bfloat16* head = reinterpret_cast<const __nv_bfloat16*>(ring_ptr + Cfg::kRingBytes);
        const int h = nt;  // weight tile = head: q heads, then k heads, then v heads
        const bool is_q = h < p.hq, is_k = !is_q && h < p.hq + p.hkv;
        const __nv_bfloat16* nw = is_q ? p.q_norm_w : p.k_norm_w;
        float nwf[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) nwf[j] = (is_q || is_k) ? __bfloat162float(nw[lane + 32 * j]) : 1.f;
        const int my_rows = p.xbox / 8;  // rows this warp handles: 4..32
        for (int i0 = 0; i0 < my_rows; i0 += 4) {
          int pos[4], dstoff_ok[4];
          __nv_bfloat16* dst[4];
          float v[4][4], cs[4][4], sn[4][4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = i0 + u;
            pos[u] = __shfl_sync(0xffffffffu, row_pos, i & 31);
            const int id = __shfl_sync(0xffffffffu, row_page, i & 31);
            const int r = (warp - 2) + 8 * i, m = m0 + r;
            dstoff_ok[u] = i < my_rows && pos[u] >= 0 && (is_q || id >= 0);
            if (dstoff_ok[u]) {
#pragma unroll
              for (int j = 0; j < 4; ++j) v[u][j] = __bfloat162float(head[r * 128 + lane + 32 * j]);
              if (is_q || is_k) {
                const __nv_bfloat16* c = p.cos_t + static_cast<size_t>(pos[u]) * 128;
                const __nv_bfloat16* sp = p.sin_t + static_cast<size_t>(pos[u]) * 128;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  cs[u][j] = __bfloat162float(c[lane + 32 * j]);
                  sn[u][j] = __bfloat162float(sp[lane + 32 * j]);
                }
              }
              if (is_q) {
                dst[u] = p.q_out + (static_cast<size_t>(m) * p.hq + h) * 128;
              } else {
                const int kvh = is_k ? h - p.hq : h - p.hq - p.hkv;
                __nv_bfloat16* pool = is_k ? p.k_pool : p.v_pool;
                dst[u] = pool + ((static_cast<size_t>(id) * p.hkv + kvh) * p.page + pos[u] % p.page) * 128;
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (!dstoff_ok[u]) continue;  // uniform across the warp
            if (is_q || is_k) {
              float ss = 0.f;
#pragma unroll
              for (int j = 0; j < 4; ++j) ss += v[u][j] * v[u][j];
              ss = warp_sum(ss);
              const float inv = rsqrtf(ss / 128.f + p.eps);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float nrm = __bfloat162float(__float2bfloat16(v[u][j] * inv));
                v[u][j] = __bfloat162float(__float2bfloat16(nwf[j] * nrm));
              }
              float rot[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int jp = (j + 2) & 3;  // partner element d +- 64 lives in the same lane
                const float other = j < 2 ? -v[u][jp] : v[u][jp];
                rot[j] = v[u][j] * cs[u][j] + other * sn[u][j];
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) v[u][j] = rot[j];
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) dst[u][lane + 32 * j] = __float2bfloat16(v[u][j]);
          }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");  // the head tile may be overwritten by the next item
      }
    }
    if (EPI == kEpiArgmax) {
      // one warp-wide maximum per row of X, once: lane l ends up with the winners of rows l, l+32, l+64, l+96
      // of this half
      uint32_t win_key[4] = {0u, 0u, 0u, 0u};
      int win_lane[4] = {0, 0, 0, 0};
#pragma unroll
      for (int j = 0; j < 128; ++j) {
        const uint32_t mx = __reduce_max_sync(0xffffffffu, best[j]);
        const unsigned who = __ballot_sync(0xffffffffu, best[j] == mx);
        if (lane == (j & 31)) {
          win_key[j >> 5] = mx;
          win_lane[j >> 5] = __ffs(who) - 1;  // equal logits of one tile: the lower feature
        }
      }
      const size_t prow = static_cast<size_t>(blockIdx.x) * 4 + quarter;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int col = half * 128 + c * 32 + lane;
        float val = -INFINITY;
        int idx = 0x7fffffff;
        if (win_key[c] != 0u) {
          const int ord = 31 - static_cast<int>(win_key[c] & 31u);     // which of this CTA's weight tiles
          const int it_of = ord / A_TILES, a_of = ord - it_of * A_TILES;
          const int tile = static_cast<int>(blockIdx.x) + it_of * static_cast<int>(gridDim.x);  // ks == 1, m_tiles == 1
          idx = (tile * A_TILES + a_of) * 128 + quarter * 32 + win_lane[c];
          val = key_float(win_key[c] & ~31u);
        }
        p.part_val[prow * kDenseMaxRows + col] = val;
        p.part_idx[prow * kDenseMaxRows + col] = idx;
      }
    }
  }

  if (EPI == kEpiStore && ks > 1) {
    // ---- split-K fold through the workspace; every thread of every CTA of the cluster joins the barrier ----
    // ks, xbox and with them rows_per are powers of two: shifts and masks, no division in the inner loops
    const int ks_shift = __ffs(ks) - 1;
    const int rows_per = p.xbox >> ks_shift;  // rows of X each CTA finishes
    const int rp_shift = __ffs(rows_per) - 1;
    const uint32_t me = cluster_ctarank();
    const int tile = static_cast<int>(blockIdx.x) >> ks_shift;
    // this tile's area: [finishing CTA r][source CTA s][rows_per][128]
    float* area = p.exchange + static_cast<size_t>(tile) * p.xbox * 128 * ks;
    if (warp >= 2) {
      const int quarter = warp & 3, half = (warp - 2) >> 2, t = quarter * 32 + lane;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      for (int c = half; c < p.xbox / 32; c += 2) {
        uint32_t v[32];
        tmem_ld32(lane_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int row = c * 32 + i;
          const int dest = row >> rp_shift, r = row & (rows_per - 1);
          // lanes hold consecutive features: one 128-byte line per warp store
          area[(((static_cast<size_t>(dest) << ks_shift) + me) << rp_shift | r) * 128 + t] = __uint_as_float(v[i]);
        }
      }
    }
    tc_fence_before();
    __syncwarp();
    cluster_sync_all();  // the partials of all CTAs of the cluster are visible to all of them
    if (warp >= 2) {
      const int tid = (warp - 2) * 32 + lane;  // 0..255
      const int nt = tile / p.m_tiles, mt = tile - nt * p.m_tiles;
      const float* mine = area + ((static_cast<size_t>(me) << ks_shift) << rp_shift) * 128;  // [source][rows_per][128]
      // (row, four features) per thread and pass; the partials of all sources are fetched together and
      // summed in rank order
      // two items per pass: the loads of both (up to 16 lines from L2) are in flight together
      for (int j0 = tid; j0 < rows_per * 32; j0 += 512) {
        float4 part[2][8];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int j = j0 + u * 256;
          if (j < rows_per * 32) {
            const int r = j >> 5, g4 = (j & 31) * 4;
#pragma unroll
            for (int src = 0; src < 8; ++src)
              if (src < ks)
                part[u][src] = __ldcg(reinterpret_cast<const float4*>(
                    mine + ((static_cast<size_t>(src) << rp_shift) + r) * 128 + g4));
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int j = j0 + u * 256;
          if (j >= rows_per * 32) break;
          const int r = j >> 5, g4 = (j & 31) * 4;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int src = 0; src < 8; ++src)
            if (src < ks) {
              acc.x += part[u][src].x;
              acc.y += part[u][src].y;
              acc.z += part[u][src].z;
              acc.w += part[u][src].w;
            }
          const int m = mt * p.xbox + static_cast<int>(me) * rows_per + r, n = nt * 128 + g4;
          if (m < p.M) {
            __nv_bfloat16* dst = p.y + static_cast<size_t>(m) * p.N + n;
            if (n + 3 < p.N && (p.N & 3) == 0) {
              uint2 o;
              o.x = pack_bf16x2(acc.x, acc.y);
              o.y = pack_bf16x2(acc.z, acc.w);
              *reinterpret_cast<uint2*>(dst) = o;
            } else {
              const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
              for (int e = 0; e < 4; ++e)
                if (n + e < p.N) dst[e] = __float2bfloat16(a4[e]);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
#endif
}

// Folds the per-warp arg-max candidates: one warp per row of X.
__global__ void __launch_bounds__(128)
argmax_fold_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int parts, int M,
                   long long* __restrict__ out) {
  grid_dep_wait();
  grid_dep_launch();
  const int m = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (m >= M) return;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int r = lane; r < parts; r += 32) {
    const float v = part_val[static_cast<size_t>(r) * kDenseMaxRows + m];
    const int i = part_idx[static_cast<size_t>(r) * kDenseMaxRows + m];
    if (v > bv || (v == bv && i < bi)) {
      bv = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if (lane == 0) out[m] = bi == 0x7fffffff ? 0 : bi;
}

static int pick_xbox(int M) {
  const int rows = M < kDenseMaxRows ? M : kDenseMaxRows;
  int box = 32;
  while (box < rows) box <<= 1;
  return box;
}

static void cluster_launch_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int grid, int smem, int ks,
                                  cudaStream_t st) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(grid);
  cfg->blockDim = dim3(kDenseThreads);
  cfg->dynamicSmemBytes = smem;
  cfg->stream = st;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ks;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
}

// How many clusters of `ks` CTAs of the split-K kernel the current device holds at once (one CTA per SM, and a
// cluster must sit inside one GPC, so this is well below SMs / ks for the larger clusters).  Asked once per
// device and size.
static int max_resident_clusters(int ks, int* out) {
  static std::mutex mu;
  static int cache[64][9];
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && cache[dev][ks] > 0) {
      *out = cache[dev][ks];
      return 0;
    }
  }
  using Cfg = DenseCfg<1>;
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&dense_gemm_kernel<1, kEpiStore>), Cfg::kSmemBytes);
  if (rc) return rc;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  cluster_launch_config(&cfg, attr, ks, Cfg::kSmemBytes, ks, nullptr);
  int n = 0;
  B200_CUDA(cudaOccupancyMaxActiveClusters(&n, dense_gemm_kernel<1, kEpiStore>, &cfg));
  if (n < 1) n = 1;
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < 64) cache[dev][ks] = n;
  *out = n;
  return 0;
}

// Shape of the launch: rows of X per work item and CTAs that share a weight tile along K.
struct DensePlan {
  int xbox, ksplit;
};

// Picks the plan with the lowest estimated time.  Per CTA: bytes pulled through TMA at about 64 B per clock,
// times the waves of CTAs when there are more items than SMs; a split adds the fp32 partial exchange (written
// and read back at about 16 B per clock, measured) and needs all its clusters resident together.
static int plan_dense(int M, int n_tiles, int k_blocks, int sms, size_t workspace_bytes, bool have_ws, DensePlan* out) {
  const int full = pick_xbox(M);
  double best = 1e30;
  out->xbox = full;
  out->ksplit = 1;
  for (int xbox = full; xbox >= 32; xbox >>= 1) {
    const int m_tiles = (M + xbox - 1) / xbox;
    const int tiles = n_tiles * m_tiles;
    for (int ks = 1; ks <= 8; ks <<= 1) {
      if (k_blocks % ks != 0 || (ks > 1 && k_blocks / ks < 4)) continue;
      if (ks > 1) {
        if (!have_ws || workspace_bytes < static_cast<size_t>(tiles) * xbox * 128 * 4 * ks) continue;
        int resident = 0;
        int rc = max_resident_clusters(ks, &resident);
        if (rc) return rc;
        if (tiles > resident) continue;
      }
      const double load = (128.0 + xbox) * (k_blocks / ks) * kDenseBlockK * 2 / 64.0;
      const int items = tiles * ks;
      const int waves = ks > 1 ? 1 : (items + sms - 1) / sms;
      const double exchange = ks > 1 ? xbox * 128.0 * 4 * 2 / 16.0 + 3000.0 : xbox * 8.0;
      const double cost = waves * load + exchange + 4000.0;
      if (cost < best) {
        best = cost;
        out->xbox = xbox;
        out->ksplit = ks;
      }
    }
    if (tiles >= 4 * sms) break;  // plenty of items already
  }
  return 0;
}

template <int A_TILES, int EPI>
static int launch_dense(const CUtensorMap& w_map, const CUtensorMap& x_map, const DenseParams& p, int grid,
                        cudaStream_t st) {
  using Cfg = DenseCfg<A_TILES, EPI>;
  const void* fn = reinterpret_cast<const void*>(&dense_gemm_kernel<A_TILES, EPI>);
  int rc = ensure_dynamic_smem(fn, Cfg::kSmemBytes);
  if (rc) return rc;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  cluster_launch_config(&cfg, attr, grid, Cfg::kSmemBytes, p.ksplit, st);
  if (overlapped_launch_enabled()) {  // the kernel holds at grid_dep_wait() after its set-up
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  B200_CUDA(cudaLaunchKernelEx(&cfg, dense_gemm_kernel<A_TILES, EPI>, w_map, x_map, p));
  return 0;
}

static int dense_args_ok(const void* x, const void* w, int M, int N, int K, const char* who) {
  B200_REQUIRE(x && w, "%s: null pointer", who);
  B200_REQUIRE(M > 0 && N > 0 && K > 0 && K % kDenseBlockK == 0, "%s: M %d, N %d, K %d (K must be a multiple of %d)",
               who, M, N, K, kDenseBlockK);
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0,
               "%s: x and w must be 16-byte aligned", who);
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_dense_gemm_workspace_bytes(int num_rows, int out_features) {
  if (num_rows <= 0 || out_features <= 0) return 0;
  // fp32 partial tiles of up to 8 K splits
  // fp32 partial tiles of up to 8 K splits; row tiles of any width cover at most the rows rounded up to 256
  const size_t rows = (static_cast<size_t>(num_rows) + kDenseMaxRows - 1) / kDenseMaxRows * kDenseMaxRows;
  const size_t n_tiles = (static_cast<size_t>(out_features) + 127) / 128;
  return rows * n_tiles * 128 * 4 * 8;
}

extern "C" int b200_dense_gemm_bf16(const void* x, const void* w, void* y, void* workspace, size_t workspace_bytes,
                                    void* status_word, int num_rows, int out_features, int in_features,
                                    int k_split, void* stream) {
  int rc = dense_args_ok(x, w, num_rows, out_features, in_features, "dense_gemm_bf16");
  if (rc) return rc;
  B200_REQUIRE(y && (reinterpret_cast<uintptr_t>(y) & 7) == 0, "dense_gemm_bf16: output must be 8-byte aligned");
  rc = check_device(nullptr);
  if (rc) return rc;
  int sms = 148;
  rc = device_sm_count(&sms);
  if (rc) return rc;
  DenseParams p{};
  p.y = static_cast<__nv_bfloat16*>(y);
  p.err = static_cast<int*>(status_word);
  p.M = num_rows;
  p.N = out_features;
  p.K = in_features;
  p.n_tiles = (out_features + 127) / 128;
  p.xbox = pick_xbox(num_rows);
  p.ksplit = k_split;
  if (k_split <= 0) {
    DensePlan plan;
    rc = plan_dense(num_rows, p.n_tiles, in_features / kDenseBlockK, sms, workspace_bytes, workspace != nullptr, &plan);
    if (rc) return rc;
    p.xbox = plan.xbox;
    p.ksplit = plan.ksplit;
  }
  p.m_tiles = (num_rows + p.xbox - 1) / p.xbox;
  B200_REQUIRE((p.ksplit == 1 || p.ksplit == 2 || p.ksplit == 4 || p.ksplit == 8) &&
                   (in_features / kDenseBlockK) % p.ksplit == 0,
               "dense_gemm_bf16: k_split %d must be 1, 2, 4 or 8 and divide the %d K blocks", p.ksplit,
               in_features / kDenseBlockK);
  if (p.ksplit > 1) {
    const size_t need = static_cast<size_t>(p.n_tiles) * p.m_tiles * p.xbox * 128 * 4 * p.ksplit;
    B200_REQUIRE(workspace && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
                 "dense_gemm_bf16: a K split needs a 16-byte aligned workspace");
    if (workspace_bytes < need) {
      set_detail("dense_gemm_bf16: workspace %zu < %zu needed for k_split %d", workspace_bytes, need, p.ksplit);
      return -kErrWorkspace;
    }
    p.exchange = static_cast<float*>(workspace);
  }
  CUtensorMap w_map, x_map;
  rc = get_tensor_map_2d(w, out_features, in_features, 2, 128, 64, &w_map);
  if (rc) return rc;
  rc = get_tensor_map_2d(x, num_rows, in_features, 2, p.xbox, 64, &x_map);
  if (rc) return rc;
  const int items = p.n_tiles * p.m_tiles * p.ksplit;
  // with a cluster every CTA has exactly one work item; without, a CTA walks items persistently
  const int grid = p.ksplit > 1 ? items : (items < sms ? items : sms);
  return launch_dense<1, kEpiStore>(w_map, x_map, p, grid, as_stream(stream));
}

extern "C" int b200_qkv_rope_append_supported(int head_dim, int in_features) {
  return head_dim == 128 && in_features > 0 && in_features % kDenseBlockK == 0;
}

extern "C" int b200_qkv_rope_append_gemm(const void* x, const void* wqkv, const void* q_norm_weight,
                                         const void* k_norm_weight, const void* cos_table, const void* sin_table,
                                         const int32_t* positions, const int32_t* block_table, void* q_out,
                                         void* k_pool, void* v_pool, void* status_word, int num_rows,
                                         int num_q_heads, int num_kv_heads, int head_dim, int in_features, float eps,
                                         int page_size, int num_blocks, int max_pages_per_seq, int max_positions,
                                         void* stream) {
  const int heads = num_q_heads + 2 * num_kv_heads;
  int rc = dense_args_ok(x, wqkv, num_rows, heads * head_dim, in_features, "qkv_rope_append_gemm");
  if (rc) return rc;
  B200_REQUIRE(q_norm_weight && k_norm_weight && cos_table && sin_table && positions && block_table && q_out && k_pool &&
                   v_pool,
               "qkv_rope_append_gemm: null pointer");
  B200_REQUIRE(b200_qkv_rope_append_supported(head_dim, in_features),
               "qkv_rope_append_gemm: head_dim %d must be 128 (one head per weight tile)", head_dim);
  B200_REQUIRE(num_q_heads > 0 && num_kv_heads > 0 && page_size > 0 && num_blocks > 0 && max_pages_per_seq > 0 &&
                   max_positions > 0,
               "qkv_rope_append_gemm: non-positive dimension");
  rc = check_device(nullptr);
  if (rc) return rc;
  int sms = 148;
  rc = device_sm_count(&sms);
  if (rc) return rc;
  DenseParams p{};
  p.err = static_cast<int*>(status_word);
  p.M = num_rows;
  p.N = heads * head_dim;
  p.K = in_features;
  p.n_tiles = heads;
  p.ksplit = 1;
  // rows per item: the width that needs the fewest waves of CTAs, then the least data per CTA
  p.xbox = pick_xbox(num_rows);
  {
    double best = 1e30;
    for (int xbox = p.xbox; xbox >= 32; xbox -= 32) {  // any multiple of 32 here: this epilogue has no K split
      const int items = heads * ((num_rows + xbox - 1) / xbox);
      const double cost = static_cast<double>((items + sms - 1) / sms) * (128.0 + xbox) + xbox * 0.25;
      if (cost < best) {
        best = cost;
        p.xbox = xbox;
      }
    }
  }
  p.m_tiles = (num_rows + p.xbox - 1) / p.xbox;
  p.q_norm_w = static_cast<const __nv_bfloat16*>(q_norm_weight);
  p.k_norm_w = static_cast<const __nv_bfloat16*>(k_norm_weight);
  p.cos_t = static_cast<const __nv_bfloat16*>(cos_table);
  p.sin_t = static_cast<const __nv_bfloat16*>(sin_table);
  p.positions = positions;
  p.block_table = block_table;
  p.q_out = static_cast<__nv_bfloat16*>(q_out);
  p.k_pool = static_cast<__nv_bfloat16*>(k_pool);
  p.v_pool = static_cast<__nv_bfloat16*>(v_pool);
  p.eps = eps;
  p.hq = num_q_heads;
  p.hkv = num_kv_heads;
  p.page = page_size;
  p.num_blocks = num_blocks;
  p.max_pages = max_pages_per_seq;
  p.max_pos = max_positions;
  CUtensorMap w_map, x_map;
  rc = get_tensor_map_2d(wqkv, p.N, in_features, 2, 128, 64, &w_map);
  if (rc) return rc;
  rc = get_tensor_map_2d(x, num_rows, in_features, 2, p.xbox, 64, &x_map);
  if (rc) return rc;
  const int items = p.n_tiles * p.m_tiles;
  return launch_dense<1, kEpiQkvRope>(w_map, x_map, p, items < sms ? items : sms, as_stream(stream));
}

extern "C" size_t b200_lm_head_argmax_workspace_bytes(void) {
  // candidates of 4 epilogue warps of up to 256 CTAs for 256 rows: value + index
  return static_cast<size_t>(256) * 4 * kDenseMaxRows * 8;
}

extern "C" int b200_lm_head_argmax(const void* x, const void* w, int64_t* next_tokens, void* workspace,
                                   size_t workspace_bytes, void* status_word, int num_rows, int vocab_size,
                                   int hidden, void* stream) {
  int rc = dense_args_ok(x, w, num_rows, vocab_size, hidden, "lm_head_argmax");
  if (rc) return rc;
  B200_REQUIRE(next_tokens && workspace, "lm_head_argmax: null pointer");
  B200_REQUIRE(num_rows <= kDenseMaxRows, "lm_head_argmax: %d rows (at most %d per call)", num_rows, kDenseMaxRows);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, "lm_head_argmax: workspace must be 16-byte aligned");
  if (workspace_bytes < b200_lm_head_argmax_workspace_bytes()) {
    set_detail("lm_head_argmax: workspace %zu < required %zu", workspace_bytes, b200_lm_head_argmax_workspace_bytes());
    return -kErrWorkspace;
  }
  rc = check_device(nullptr);
  if (rc) return rc;
  int sms = 148;
  rc = device_sm_count(&sms);
  if (rc) return rc;
  DenseParams p{};
  p.err = static_cast<int*>(status_word);
  p.M = num_rows;
  p.N = vocab_size;
  p.K = hidden;
  p.m_tiles = 1;
  p.n_tiles = (vocab_size + 255) / 256;
  p.xbox = pick_xbox(num_rows);
  p.ksplit = 1;
  const int grid = p.n_tiles < sms ? p.n_tiles : (sms < 256 ? sms : 256);
  B200_REQUIRE((p.n_tiles + grid - 1) / grid <= 16, "lm_head_argmax: vocabulary of %d needs more than 32 weight tiles "
               "per CTA on this device", vocab_size);
  p.part_val = static_cast<float*>(workspace);
  p.part_idx = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + static_cast<size_t>(256) * 4 * kDenseMaxRows * 4);
  CUtensorMap w_map, x_map;
  rc = get_tensor_map_2d(w, vocab_size, hidden, 2, 128, 64, &w_map);
  if (rc) return rc;
  rc = get_tensor_map_2d(x, num_rows, hidden, 2, p.xbox, 64, &x_map);
  if (rc) return rc;
  rc = launch_dense<2, kEpiArgmax>(w_map, x_map, p, grid, as_stream(stream));
  if (rc) return rc;
  B200_CUDA(launch_overlapped(argmax_fold_kernel, dim3((num_rows + 3) / 4), dim3(128), 0, as_stream(stream), p.part_val,
                              p.part_idx, grid * 4, num_rows, reinterpret_cast<long long*>(next_tokens)));
  return 0;
}
