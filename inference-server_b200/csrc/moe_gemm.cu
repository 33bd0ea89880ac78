// FP8 (e4m3) block-scaled grouped GEMM for the MoE expert layer, sm_100a.
//
// Computes what the reference's model forward does per expert
// (src/inference_server/backends/torch_backend.py:305-322 -> transformers
// expert forward): [g;u] = W13 x, h = silu(g) * u, y = W2 h, on weights stored
// as e4m3 with one fp32 scale per 128x128 tile and activations stored as e4m3
// with one fp32 scale per row per 128 columns:
//     C[r, n] = sum_kb  a_scale[r, kb] * w_scale[n / 128, kb]
//                       * sum_{k in kb} A[r, k] * W[n, k]
//
// One persistent CTA per SM, 3 warpgroups (12 warps).  Warpgroup 0 holds the two
// single-thread roles and gives most of its registers back (setmaxnreg) so that
// the 8 promotion warps can hold 128 accumulators plus two TMEM loads in flight:
//   warp 0      TMA producer: per 128-wide K block one A box (the tile's sorted rows x
//               128 B; 32, 64 or 128 rows, whichever first covers the tile, so a decode
//               batch with a dozen rows per expert does not pull 128 through the ring)
//               and two W boxes (128 rows x 128 B each) into a 4-stage ring, 128-byte
//               swizzle, completion by mbarrier bytes.
//   warp 1      MMA issuer: one thread issues 4 x tcgen05.mma (M128 N256 K32,
//               kind::f8f6f4) per K block into one of two 256-column TMEM
//               accumulators and commits to the stage-empty and
//               accumulator-full barriers.
//   warps 4-11  promotion + epilogue: each thread owns one row and 128 of the 256
//               columns; per K block it reads the raw block sum from TMEM
//               (tcgen05.ld 32x32b), multiplies by the two scales and adds into
//               fp32 registers, then frees the accumulator.  fp32 block scales
//               are not expressible in the tensor-core block-scaled formats, so
//               this promotion runs on the CUDA cores while the next K block is
//               in the tensor pipe.
//   gate/up     tile columns = 128 gate rows + the matching 128 up rows of W13,
//               so SwiGLU and the per-row amax over the 128 outputs stay inside
//               two threads; h is written as e4m3 + scale, ready for the down GEMM.
//   down        tile columns = 256 rows of W2; writes bf16 rows in sorted order.
// SwiGLU is evaluated in fp32 on the fp32 accumulators and quantised directly.
// A tile is 128 consecutive sorted rows of one expert (see MoeTile); rows past
// the expert's count are computed on whatever the box holds and never stored.

#include "common.cuh"
#include "host.h"

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
  // bounds the tile list is checked against: a stale or foreign list must not steer a load or a store
  int num_rows, num_experts, max_tiles;
};

// A tile record is usable when it names an existing expert and rows inside the activation matrix.  All three
// roles of the kernel evaluate this on the same record and skip the same tiles, so their ring and accumulator
// counters stay in step.
__device__ __forceinline__ bool tile_ok(const MoeTile& t, const GemmParams& p) {
  return t.expert >= 0 && t.expert < p.num_experts && t.rows > 0 && t.rows <= kTileM && t.row0 >= 0 &&
         t.row0 + t.rows <= p.num_rows;
}

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
moe_fp8_gemm_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap a_map64,
                    const __grid_constant__ CUtensorMap a_map32, const __grid_constant__ CUtensorMap b_map,
                    const GemmParams p) {
#ifdef B200_DEVICE_OK
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
  const uint32_t bars = ring + kGemmStages * kStageBytesG;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kGemmStages;
  const uint32_t bar_tfull = bars + 16 * kGemmStages, bar_tempty = bar_tfull + 16;
  const uint32_t bar_amax = bar_tempty + 16;
  uint32_t* tmem_base_sm = reinterpret_cast<uint32_t*>(ring_ptr + kGemmStages * kStageBytesG + 128);
  float* amax_sm = reinterpret_cast<float*>(ring_ptr + kGemmStages * kStageBytesG + 144);  // [2][2][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGemmStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, kEpiWarps);
      mbar_init(bar_amax + 8 * s, kEpiWarps);
    }
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_base_sm), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_sm;
  // Set-up done; the tile list, the activations and their scales come from the kernels before this one.
  grid_dep_wait();
  grid_dep_launch();

  int listed = *p.num_tiles;
  if (listed < 0 || listed > p.max_tiles) {
    if (threadIdx.x == 0) set_error(p.err, kErrDevBadExpert);
    listed = listed < 0 ? 0 : p.max_tiles;
  }
  const int total = listed * p.n_tiles;

  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    // ------------------------------------------------------------ TMA ------
    if (lane == 0) {
      tma_prefetch_desc(&a_map);
      tma_prefetch_desc(&a_map64);
      tma_prefetch_desc(&a_map32);
      tma_prefetch_desc(&b_map);
      uint32_t it = 0;
      bool alive = true;
      for (int w = blockIdx.x; w < total && alive; w += gridDim.x) {
        const MoeTile tile = p.tiles[w / p.n_tiles];
        if (!tile_ok(tile, p)) {
          set_error(p.err, kErrDevBadExpert);
          continue;
        }
        const int j = w % p.n_tiles;
        // the two 128-row blocks of W this tile multiplies with: block index inside the expert
        int nb0, nb1;
        if (MODE == kModeGateUp) {
          nb0 = j;
          nb1 = p.inter / 128 + j;
        } else {
          nb0 = 2 * j;
          nb1 = 2 * j + 1;
        }
        const int sblocks = p.n_rows / 128;
        // row-major weights: block (nb, kb) starts at row expert*n_rows + nb*128, column kb*128;
        // tiled weights: it is the contiguous 16 KiB block number (expert*sblocks + nb)*k_blocks + kb
        const int b_row0 = p.tiled ? (tile.expert * sblocks + nb0) * p.k_blocks * 128 : tile.expert * p.n_rows + nb0 * 128;
        const int b_row1 = p.tiled ? (tile.expert * sblocks + nb1) * p.k_blocks * 128 : tile.expert * p.n_rows + nb1 * 128;
        // The A box only needs the tile's own rows.  The MMA still reads 128 rows of the stage; what an earlier
        // tile left in the rows below the box only reaches accumulator rows that are never stored.
        const CUtensorMap* amap = tile.rows <= 32 ? &a_map32 : (tile.rows <= 64 ? &a_map64 : &a_map);
        const uint32_t stage_bytes = (tile.rows <= 32 ? 32u : (tile.rows <= 64 ? 64u : 128u)) * kBlockK + kBBytes;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t slot = it % kGemmStages, phase = (it / kGemmStages) & 1;
          alive = mbar_wait(bar_empty + 8 * slot, phase ^ 1, p.err);
          if (!alive) break;
          const uint32_t sa = ring + slot * kStageBytesG, sb = sa + kABytes;
          mbar_arrive_expect_tx(bar_full + 8 * slot, stage_bytes);
          tma_load_2d(sa, amap, bar_full + 8 * slot, kb * kBlockK, tile.row0);
          const int bx = p.tiled ? 0 : kb * kBlockK, by = p.tiled ? kb * 128 : 0;
          tma_load_2d(sb, &b_map, bar_full + 8 * slot, bx, b_row0 + by);
          tma_load_2d(sb + kBBytes / 2, &b_map, bar_full + 8 * slot, bx, b_row1 + by);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA ------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f8(kTileM, kTileN);
      uint32_t it = 0;
      bool alive = true;
      for (int w = blockIdx.x; w < total && alive; w += gridDim.x) {
        if (!tile_ok(p.tiles[w / p.n_tiles], p)) continue;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t slot = it % kGemmStages, phase = (it / kGemmStages) & 1;
          const uint32_t buf = it & 1, aphase = (it >> 1) & 1;
          alive = mbar_wait(bar_full + 8 * slot, phase, p.err);
          alive = alive && mbar_wait(bar_tempty + 8 * buf, aphase ^ 1, p.err);
          if (!alive) break;
          tc_fence_after();
          const uint32_t sa = ring + slot * kStageBytesG, sb = sa + kABytes;
          const uint64_t a_desc = umma_desc_k128(sa), b_desc = umma_desc_k128(sb);
          const uint32_t d = tmem_base + buf * kTileN;
#pragma unroll
          for (int k = 0; k < kBlockK / 32; ++k)
            tc_mma_f8(d, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
          tc_commit(bar_empty + 8 * slot);
          tc_commit(bar_tfull + 8 * buf);
        }
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ------------------------------------------- promotion + epilogue ------
    const int quarter = warp & 3;        // TMEM lane quarter this warp may read
    const int half = (warp - 4) >> 2;    // which 128 of the tile's 256 columns
    const int r = quarter * 32 + lane;   // row inside the tile
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    uint32_t it = 0, tile_it = 0;
    bool alive = true;
    for (int w = blockIdx.x; w < total && alive; w += gridDim.x) {
      const MoeTile tile = p.tiles[w / p.n_tiles];
      if (!tile_ok(tile, p)) continue;
      const int j = w % p.n_tiles;
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
        alive = mbar_wait(bar_tfull + 8 * buf, aphase, p.err);
        if (!alive) break;
        tc_fence_after();
        const uint32_t t0 = lane_addr + buf * kTileN;
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
            if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
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
      }
      if (!alive) break;

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
        float* ax = amax_sm + (tile_it & 1) * 2 * kTileM;
        ax[half * kTileM + r] = amax;
        // The partner thread (same row, other column half) holds the rest of the
        // 128-wide quantisation group; exchange through shared memory.  The
        // buffers and barriers alternate per tile so a slow reader of tile i
        // cannot see the writes of tile i + 2.
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_amax + 8 * (tile_it & 1));
        alive = mbar_wait(bar_amax + 8 * (tile_it & 1), (tile_it >> 1) & 1, p.err);
        if (!alive) break;
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
      ++tile_it;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
#endif
}

// The three A maps: boxes of 128, 64 and 32 rows over the same activation matrix.
struct AMaps {
  CUtensorMap m128, m64, m32;
};
static int make_a_maps(const void* a, int rows, int cols, AMaps* out) {
  int rc = get_tensor_map_2d(a, rows, cols, 1, 128, 128, &out->m128);
  if (rc) return rc;
  rc = get_tensor_map_2d(a, rows, cols, 1, 64, 128, &out->m64);
  if (rc) return rc;
  return get_tensor_map_2d(a, rows, cols, 1, 32, 128, &out->m32);
}

template <int MODE>
static int launch_gemm(const AMaps& a, const CUtensorMap& b_map, const GemmParams& p,
                       cudaStream_t st) {
  int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&moe_fp8_gemm_kernel<MODE>), kGemmSmem);
  if (rc) return rc;
  int grid = 148;
  rc = device_sm_count(&grid);
  if (rc) return rc;
  B200_CUDA(launch_overlapped(moe_fp8_gemm_kernel<MODE>, dim3(grid), dim3(kGemmThreads), kGemmSmem, st, a.m128, a.m64,
                              a.m32, b_map, p));
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200

using namespace b200;

static int aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int b200_moe_fp8_gemm_gate_up(const void* xq, const float* x_scale, const void* w13,
                                         const float* w13_scale_inv, const void* tiles,
                                         const int32_t* num_tiles, void* hq, float* h_scale,
                                         void* status_word, int num_rows, int num_experts,
                                         int hidden, int inter, int weight_layout, void* stream) {
  B200_REQUIRE(xq && x_scale && w13 && w13_scale_inv && tiles && num_tiles && hq && h_scale,
               "moe_fp8_gemm_gate_up: null pointer");
  B200_REQUIRE(num_rows >= 0 && num_experts > 0, "moe_fp8_gemm_gate_up: bad row/expert count");
  B200_REQUIRE(hidden > 0 && hidden % 128 == 0 && inter > 0 && inter % 128 == 0,
               "moe_fp8_gemm_gate_up: hidden %d and inter %d must be multiples of 128", hidden, inter);
  B200_REQUIRE(aligned16(xq) && aligned16(w13) && aligned16(hq),
               "moe_fp8_gemm_gate_up: buffers must be 16-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  if (num_rows == 0) return 0;
  AMaps a_map;
  CUtensorMap b_map;
  rc = make_a_maps(xq, num_rows, hidden, &a_map);
  if (rc) return rc;
  B200_REQUIRE(weight_layout == 0 || weight_layout == 1, "moe_fp8_gemm_gate_up: weight_layout %d is neither 0 nor 1",
               weight_layout);
  if (weight_layout == 1)
    rc = get_tensor_map_2d(w13, static_cast<uint64_t>(num_experts) * 2 * inter * (hidden / 128), 128, 1, 128, 128, &b_map);
  else
    rc = get_tensor_map_2d(w13, static_cast<uint64_t>(num_experts) * 2 * inter, hidden, 1, 128, 128, &b_map);
  if (rc) return rc;
  GemmParams p{};
  p.a_scale = x_scale;
  p.b_scale = w13_scale_inv;
  p.tiles = static_cast<const MoeTile*>(tiles);
  p.num_tiles = num_tiles;
  p.hq = static_cast<uint8_t*>(hq);
  p.hs = h_scale;
  p.err = static_cast<int*>(status_word);
  p.k_blocks = hidden / 128;
  p.n_rows = 2 * inter;
  p.inter = inter;
  p.n_tiles = inter / 128;
  p.tiled = weight_layout;
  p.num_rows = num_rows;
  p.num_experts = num_experts;
  p.max_tiles = (num_rows + kTileM - 1) / kTileM + num_experts;
  return launch_gemm<kModeGateUp>(a_map, b_map, p, as_stream(stream));
}

static int gemm_down_impl(const void* hq, const float* h_scale, const void* w2, const float* w2_scale_inv,
                          const void* tiles, const int32_t* num_tiles, void* y_sorted,
                          const int32_t* out_row_map, void* status_word, int num_rows, int num_experts,
                          int hidden, int inter, int weight_layout, void* const* y_peers, int ep_world,
                          int ep_capacity, int ep_rank, void* stream) {
  B200_REQUIRE(hq && h_scale && w2 && w2_scale_inv && tiles && num_tiles && (y_sorted || y_peers),
               "moe_fp8_gemm_down: null pointer");
  B200_REQUIRE(num_rows >= 0 && num_experts > 0, "moe_fp8_gemm_down: bad row/expert count");
  B200_REQUIRE(hidden > 0 && hidden % 256 == 0 && inter > 0 && inter % 128 == 0,
               "moe_fp8_gemm_down: hidden %d must be a multiple of 256 and inter %d of 128", hidden, inter);
  B200_REQUIRE(aligned16(hq) && aligned16(w2) && (y_sorted == nullptr || aligned16(y_sorted)),
               "moe_fp8_gemm_down: buffers must be 16-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  if (num_rows == 0) return 0;
  AMaps a_map;
  CUtensorMap b_map;
  rc = make_a_maps(hq, num_rows, inter, &a_map);
  if (rc) return rc;
  B200_REQUIRE(weight_layout == 0 || weight_layout == 1, "moe_fp8_gemm_down: weight_layout %d is neither 0 nor 1",
               weight_layout);
  if (weight_layout == 1)
    rc = get_tensor_map_2d(w2, static_cast<uint64_t>(num_experts) * hidden * (inter / 128), 128, 1, 128, 128, &b_map);
  else
    rc = get_tensor_map_2d(w2, static_cast<uint64_t>(num_experts) * hidden, inter, 1, 128, 128, &b_map);
  if (rc) return rc;
  GemmParams p{};
  p.a_scale = h_scale;
  p.b_scale = w2_scale_inv;
  p.tiles = static_cast<const MoeTile*>(tiles);
  p.num_tiles = num_tiles;
  p.y = static_cast<__nv_bfloat16*>(y_sorted);
  p.out_row_map = out_row_map;
  p.err = static_cast<int*>(status_word);
  p.k_blocks = inter / 128;
  p.n_rows = hidden;
  p.inter = inter;
  p.n_tiles = hidden / kTileN;
  p.tiled = weight_layout;
  p.num_rows = num_rows;
  p.num_experts = num_experts;
  p.max_tiles = (num_rows + kTileM - 1) / kTileM + num_experts;
  if (y_peers != nullptr) {
    B200_REQUIRE(ep_world >= 1 && ep_world <= kMaxEpWorld && ep_capacity > 0 && ep_rank >= 0 && ep_rank < ep_world &&
                     out_row_map != nullptr,
                 "moe_fp8_gemm_down_p2p: world %d (at most %d), capacity %d, rank %d, row map %p", ep_world,
                 kMaxEpWorld, ep_capacity, ep_rank, static_cast<const void*>(out_row_map));
    for (int r = 0; r < ep_world; ++r) {
      B200_REQUIRE(y_peers[r] && aligned16(y_peers[r]), "moe_fp8_gemm_down_p2p: buffer of rank %d null or unaligned", r);
      p.y_peers[r] = static_cast<__nv_bfloat16*>(y_peers[r]);
    }
    p.peer_capacity = ep_capacity;
    p.my_rank = ep_rank;
  }
  return launch_gemm<kModeDown>(a_map, b_map, p, as_stream(stream));
}

extern "C" int b200_moe_fp8_gemm_down(const void* hq, const float* h_scale, const void* w2,
                                      const float* w2_scale_inv, const void* tiles,
                                      const int32_t* num_tiles, void* y_sorted,
                                      const int32_t* out_row_map, void* status_word,
                                      int num_rows, int num_experts, int hidden, int inter,
                                      int weight_layout, void* stream) {
  B200_REQUIRE(y_sorted, "moe_fp8_gemm_down: null pointer");
  return gemm_down_impl(hq, h_scale, w2, w2_scale_inv, tiles, num_tiles, y_sorted, out_row_map, status_word,
                        num_rows, num_experts, hidden, inter, weight_layout, nullptr, 0, 0, 0, stream);
}

extern "C" int b200_moe_fp8_gemm_down_p2p(const void* hq, const float* h_scale, const void* w2,
                                          const float* w2_scale_inv, const void* tiles,
                                          const int32_t* num_tiles, void* const* y_peers,
                                          const int32_t* out_row_map, void* status_word, int num_rows,
                                          int num_experts, int hidden, int inter, int weight_layout,
                                          int ep_world, int ep_capacity, int ep_rank, void* stream) {
  B200_REQUIRE(y_peers, "moe_fp8_gemm_down_p2p: null pointer");
  return gemm_down_impl(hq, h_scale, w2, w2_scale_inv, tiles, num_tiles, nullptr, out_row_map, status_word,
                        num_rows, num_experts, hidden, inter, weight_layout, y_peers, ep_world, ep_capacity,
                        ep_rank, stream);
}
