// Pieces shared by the two forms of the FP8 block-scaled grouped GEMM (one CTA per tile: moe_gemm.cu; a CTA
// pair per two row tiles of one expert: moe_gemm_pair.cu): tile geometry, kernel parameters, and the work of
// the promotion warps for one tile - per 128-wide K block read the raw block sum from TMEM, scale it and add
// it into fp32 registers, then the epilogue (SwiGLU + e4m3 re-quantisation, or bf16 rows out).
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kGemmStages = 4;
constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kBlockK = 128;
constexpr int kABytes = kTileM * kBlockK;
constexpr int kBBytes = kTileN * kBlockK;
constexpr int kStageBytesG = kABytes + kBBytes;
constexpr int kEpiWarps = 8;
constexpr int kGemmThreads = (4 + kEpiWarps) * 32;  // warps 2, 3 idle: roles are per warpgroup
constexpr int kTmemCols = 512;
constexpr int kGemmSmem = kGemmStages * kStageBytesG + 1024 /* align */ + 128 /* barriers */ +
                          16 /* tmem base */ + 2 * 2 * kTileM * 4 /* amax exchange */;

enum : int { kModeGateUp = 0, kModeDown = 1 };

// Optional timeline trace for tuning: compiled in only with -DB200_GEMM_TRACE.
#ifdef B200_GEMM_TRACE
__device__ long long* g_gemm_trace = nullptr;  // [role 0..3][4096] clock64 stamps of CTA 0
#define B200_TRACE(role, idx)                                                         \
  do {                                                                                \
    if (blockIdx.x == 0 && g_gemm_trace != nullptr && (idx) < 4096)                   \
      g_gemm_trace[(role) * 4096 + (idx)] = clock64();                                \
  } while (0)
#else
#define B200_TRACE(role, idx) do { } while (0)
#endif

struct GemmParams {
  const float* a_scale;  // [rows, k_blocks]
  const float* b_scale;  // [E, n_rows / 128, k_blocks]
  const MoeTile* tiles;
  const int* num_tiles;
  uint8_t* hq;           // gate/up: [rows, inter] e4m3
  float* hs;             // gate/up: [rows, inter / 128]
  __nv_bfloat16* y;      // down:    [rows, n_rows]
  const int* out_row_map;  // down: output row of each sorted row, or null for the identity
  int* err;
  int k_blocks;          // K / 128
  int n_rows;            // weight rows per expert (2 * inter, or hidden)
  int inter;             // gate/up only
  int n_tiles;           // column tiles per row tile
  int tiled;             // weights stored as contiguous 128x128 blocks [E, n_rows/128, k_blocks, 128, 128]
  // down, expert-parallel return path: output row o = r * peer_capacity + i (slot i received from rank r) is
  // written to row my_rank * peer_capacity + i of rank r's buffer y_peers[r] instead of to y.  Off when
  // peer_capacity is 0.
  __nv_bfloat16* y_peers[kMaxEpWorld];
  int peer_capacity;
  int my_rank;
};

// Host side of the CTA-pair form (moe_gemm_pair.cu).  mode: kModeGateUp or kModeDown.
int launch_gemm_pair(int mode, const CUtensorMap& a_map, const CUtensorMap& b_map, const GemmParams& p,
                     cudaStream_t st);
int gemm_pair_max_tiles();

// What a promotion thread needs to know about its CTA.
struct PromoCtx {
  uint32_t bar_tfull;   // accumulator-full barriers of this CTA (2)
  uint32_t bar_tempty;  // accumulator-empty barriers the MMA issuer waits on: a shared::cta address, or with
                        // REMOTE_TEMPTY a shared::cluster address in the CTA that issues the MMAs
  uint32_t bar_amax;    // amax exchange barriers of this CTA (2)
  float* amax_sm;       // [2][2][128]
  uint32_t lane_addr;   // TMEM address of this warp's lane quarter, column 0
  int half;             // which 128 of the tile's 256 columns this thread owns
  int r;                // row inside the tile = TMEM lane
  int lane;
};

// One tile (row tile `tile` of its expert x column tile j) on the promotion side: K loop, then epilogue.
// `it` counts K blocks and `tile_it` tiles since the kernel started (barrier phases).  Returns false when a
// bounded wait ran out.
template <int MODE, bool REMOTE_TEMPTY>
__device__ __forceinline__ bool promo_tile(const GemmParams& p, const PromoCtx& cx, const MoeTile& tile, int j,
                                           uint32_t& it, uint32_t tile_it) {
  const int half = cx.half, r = cx.r, lane = cx.lane;
  const bool row_ok = r < tile.rows;
  const size_t grow = static_cast<size_t>(tile.row0) + r;
  const float* as = p.a_scale + grow * p.k_blocks;
  const int sblocks = p.n_rows / 128;
  const float *bs0, *bs1;
  if (MODE == kModeGateUp) {
    bs0 = p.b_scale + (static_cast<size_t>(tile.expert) * sblocks + j) * p.k_blocks;
    bs1 = bs0 + static_cast<size_t>(p.inter / 128) * p.k_blocks;
  } else {
    bs0 = p.b_scale + (static_cast<size_t>(tile.expert) * sblocks + 2 * j + half) * p.k_blocks;
    bs1 = bs0;
  }
  float acc[128];
#pragma unroll
  for (int i = 0; i < 128; ++i) acc[i] = 0.f;

  for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
    const uint32_t buf = it & 1, aphase = (it >> 1) & 1;
    const float sa = row_ok ? __ldg(as + kb) : 0.f;
    const float s0 = sa * __ldg(bs0 + kb), s1 = sa * __ldg(bs1 + kb);
    if (!mbar_wait(cx.bar_tfull + 8 * buf, aphase, p.err)) return false;
    if (threadIdx.x == 128) B200_TRACE(2, 2 * it);
    tc_fence_after();
    const uint32_t t0 = cx.lane_addr + buf * kTileN;
#pragma unroll
    for (int c = 0; c < 4; c += 2) {
      uint32_t col0, col1;
      float sc0, sc1;
      if (MODE == kModeGateUp) {
        col0 = (c < 2 ? 0 : 128) + half * 64;
        col1 = col0 + 32;
        sc0 = sc1 = c < 2 ? s0 : s1;
      } else {
        col0 = half * 128 + c * 32;
        col1 = col0 + 32;
        sc0 = sc1 = s0;
      }
      uint32_t v0[32], v1[32];
      tmem_ld32(t0 + col0, v0);
      tmem_ld32(t0 + col1, v1);
      tmem_ld_wait();
      if (c == 2) {
        // everything this thread needs from the accumulator is in registers
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (REMOTE_TEMPTY) mbar_arrive_cluster(cx.bar_tempty + 8 * buf);
          else mbar_arrive(cx.bar_tempty + 8 * buf);
        }
      }
      // packed fp32 FMA (two lanes per instruction) halves the issue slots of the promotion
      const float2 sc0v = make_float2(sc0, sc0), sc1v = make_float2(sc1, sc1);
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const float2 r0 = __ffma2_rn(make_float2(__uint_as_float(v0[i]), __uint_as_float(v0[i + 1])), sc0v,
                                     make_float2(acc[c * 32 + i], acc[c * 32 + i + 1]));
        acc[c * 32 + i] = r0.x;
        acc[c * 32 + i + 1] = r0.y;
        const float2 r1 = __ffma2_rn(make_float2(__uint_as_float(v1[i]), __uint_as_float(v1[i + 1])), sc1v,
                                     make_float2(acc[c * 32 + 32 + i], acc[c * 32 + 32 + i + 1]));
        acc[c * 32 + 32 + i] = r1.x;
        acc[c * 32 + 32 + i + 1] = r1.y;
      }
    }
    if (threadIdx.x == 128) B200_TRACE(2, 2 * it + 1);
  }
  if (threadIdx.x == 128) B200_TRACE(3, 4 * tile_it);

  if (MODE == kModeGateUp) {
    // acc[0..63] = gate, acc[64..127] = up for inter columns j*128 + half*64 + i
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      const float g = acc[i];
      // silu(g) = g * sigmoid(g) = 0.5 g (1 + tanh(g / 2)): one special-function op per element instead of
      // two (exp + reciprocal); the loop is bound by that unit.  tanh.approx is good to ~2^-11 relative.
      float th;
      asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * g));
      const float h = (0.5f * g) * (1.f + th) * acc[64 + i];
      acc[i] = h;
      amax = fmaxf(amax, fabsf(h));
    }
    if (threadIdx.x == 128) B200_TRACE(3, 4 * tile_it + 1);
    float* ax = cx.amax_sm + (tile_it & 1) * 2 * kTileM;
    ax[half * kTileM + r] = amax;
    // The partner thread (same row, other column half) holds the rest of the
    // 128-wide quantisation group; exchange through shared memory.  The
    // buffers and barriers alternate per tile so a slow reader of tile i
    // cannot see the writes of tile i + 2.
    __syncwarp();
    if (lane == 0) mbar_arrive(cx.bar_amax + 8 * (tile_it & 1));
    if (!mbar_wait(cx.bar_amax + 8 * (tile_it & 1), (tile_it >> 1) & 1, p.err)) return false;
    if (threadIdx.x == 128) B200_TRACE(3, 4 * tile_it + 2);
    amax = fmaxf(amax, ax[(half ^ 1) * kTileM + r]);
    const float s = amax > 0.f ? amax / 448.f : 1.f;
    const float inv_s = 1.f / s;
    if (row_ok) {
      uint8_t* dst = p.hq + grow * p.inter + j * 128 + half * 64;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t wd[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int b = c * 16 + q * 4;
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(acc[b] * inv_s, acc[b + 1] * inv_s),
                                                       __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(acc[b + 2] * inv_s, acc[b + 3] * inv_s),
                                                       __NV_SATFINITE, __NV_E4M3);
          wd[q] = lo | (hi << 16);
        }
        *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
      }
      if (half == 0) p.hs[grow * (p.inter / 128) + j] = s;
    }
  } else {
    if (row_ok) {
      size_t orow = p.out_row_map ? static_cast<size_t>(__ldg(p.out_row_map + grow)) : grow;
      __nv_bfloat16* ybase = p.y;
      if (p.peer_capacity > 0) {
        const int src = static_cast<int>(orow) / p.peer_capacity;
        orow = static_cast<size_t>(p.my_rank) * p.peer_capacity + (orow - static_cast<size_t>(src) * p.peer_capacity);
        ybase = p.y_peers[src];
      }
      __nv_bfloat16* dst = ybase + orow * p.n_rows + j * kTileN + half * 128;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint4 o;
        o.x = pack_bf16x2(acc[c * 8 + 0], acc[c * 8 + 1]);
        o.y = pack_bf16x2(acc[c * 8 + 2], acc[c * 8 + 3]);
        o.z = pack_bf16x2(acc[c * 8 + 4], acc[c * 8 + 5]);
        o.w = pack_bf16x2(acc[c * 8 + 6], acc[c * 8 + 7]);
        *reinterpret_cast<uint4*>(dst + c * 8) = o;
      }
    }
  }
  if (threadIdx.x == 128) B200_TRACE(3, 4 * tile_it + 3);
  return true;
}

}  // namespace b200
