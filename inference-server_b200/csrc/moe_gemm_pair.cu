// CTA-pair form of the FP8 block-scaled grouped GEMM (tcgen05 cta_group::2), for many rows per expert.
//
// With one CTA per 128 x 256 tile (moe_gemm.cu) every CTA re-reads a 16 KiB A block and a 32 KiB W block per
// 128-wide K block, and at thousands of tokens the kernel is bound by that L2 -> SM operand stream, not by the
// tensor pipe.  Here two CTAs of a cluster, on the two SMs of a pair, take TWO row tiles of the same expert
// against ONE column tile of its weights: one tcgen05.mma of M = 256 per K = 32 slice, issued by the even CTA,
// in which each CTA supplies its own 128 rows of A and HALF of the W rows (the even CTA the first 128-row block
// of the tile, the odd CTA the second), and keeps the 128 x 256 accumulator of its own rows in its own TMEM.
// Per CTA and K block that is 16 KiB + 16 KiB instead of 16 KiB + 32 KiB, and six 32 KiB stages fit.
//
// Roles per CTA are those of moe_gemm.cu (warp 0 TMA, warp 1 MMA - idle in the odd CTA -, warps 4-11 promotion
// and epilogue on the CTA's own rows); the arithmetic per element is identical.  Barriers:
//   full[s]    in the even CTA only: its producer expects the bytes of BOTH CTAs, both CTAs' loads complete on it
//   empty[s]   in each CTA: the issuer commits to its own and to the odd CTA's
//   tfull[b]   in each CTA: the issuer commits to both
//   tempty[b]  in the even CTA: 8 promotion warps of each CTA arrive (the odd CTA's across the cluster)
// An expert with an odd number of row tiles leaves the odd CTA of its last pair without rows: it computes on
// whatever its A box holds and stores nothing.  The pairs are found from the row-tile list in the prologue
// (MoeTile.pad holds the tile's ordinal inside its expert).
#include "common.cuh"
#include "host.h"
#include "moe_gemm.cuh"

namespace b200 {

constexpr int kPairStages = 6;
constexpr int kPairStageBytes = kABytes + kBBytes / 2;  // A block + one W block
constexpr int kPairMaxPairs = 1536;                     // pair list in shared memory (uint16 each)
constexpr int kPairSmem = kPairStages * kPairStageBytes + 1024 /* align */ + 256 /* barriers */ + 16 /* tmem base */ +
                          2 * 2 * kTileM * 4 /* amax exchange */ + kPairMaxPairs * 2 + 16;

template <int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
moe_fp8_gemm_pair_kernel(const __grid_constant__ CUtensorMap a_map,
                         const __grid_constant__ CUtensorMap b_map, const GemmParams p) {
#ifdef B200_DEVICE_OK
  extern __shared__ uint8_t smem_raw[];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
  constexpr int kRing = kPairStages * kPairStageBytes;
  const uint32_t bars = ring + kRing;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kPairStages;
  const uint32_t bar_tfull = bars + 16 * kPairStages, bar_tempty = bar_tfull + 16;
  const uint32_t bar_amax = bar_tempty + 16;
  uint32_t* tmem_base_sm = reinterpret_cast<uint32_t*>(ring_ptr + kRing + 256);
  float* amax_sm = reinterpret_cast<float*>(ring_ptr + kRing + 272);  // [2][2][128]
  uint16_t* pair_first = reinterpret_cast<uint16_t*>(ring_ptr + kRing + 272 + 2 * 2 * kTileM * 4);
  int* num_pairs_sm = reinterpret_cast<int*>(pair_first + kPairMaxPairs);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = even CTA (issues the MMAs), 1 = odd CTA
  const int pair_id = blockIdx.x >> 1, n_pair_ctas = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, 2 * kEpiWarps);
      mbar_init(bar_amax + 8 * s, kEpiWarps);
    }
    fence_mbar_init();
    fence_proxy_async();
    // pairs: a row tile with an even ordinal inside its expert starts one; its partner is the next tile if that
    // belongs to the same expert
    const int nt = *p.num_tiles;
    int np = 0;
    for (int t = 0; t < nt && np < kPairMaxPairs; ++t)
      if ((p.tiles[t].pad & 1) == 0) pair_first[np++] = static_cast<uint16_t>(t);
    *num_pairs_sm = np;
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(tmem_base_sm), kTmemCols);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the other CTA's barriers exist before anything is signalled across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_sm;
  const int num_tiles = *p.num_tiles;
  const int total = (*num_pairs_sm) * p.n_tiles;

  // this CTA's row tile of work item w (a tile with rows = 0 when the pair has no second tile)
  auto my_tile = [&](int w) {
    const int first = pair_first[w / p.n_tiles];
    MoeTile t = p.tiles[first];
    if (rank == 1) {
      const bool has = first + 1 < num_tiles && p.tiles[first + 1].expert == t.expert;
      if (has) t = p.tiles[first + 1];
      else t.rows = 0;
    }
    return t;
  };

  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    // ------------------------------------------------------------ TMA ------
    if (lane == 0) {
      tma_prefetch_desc(&a_map);
      tma_prefetch_desc(&b_map);
      uint32_t it = 0;
      bool alive = true;
      for (int w = pair_id; w < total && alive; w += n_pair_ctas) {
        const MoeTile tile = my_tile(w);
        const int j = w % p.n_tiles;
        // this CTA's 128-row block of W: the even CTA the tile's first block, the odd CTA its second
        int nb;
        if (MODE == kModeGateUp) nb = rank == 0 ? j : p.inter / 128 + j;
        else nb = 2 * j + static_cast<int>(rank);
        const int sblocks = p.n_rows / 128;
        const int b_row = p.tiled ? (tile.expert * sblocks + nb) * p.k_blocks * 128 : tile.expert * p.n_rows + nb * 128;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t slot = it % kPairStages, phase = (it / kPairStages) & 1;
          alive = mbar_wait(bar_empty + 8 * slot, phase ^ 1, p.err);
          if (!alive) break;
          const uint32_t sa = ring + slot * kPairStageBytes, sb = sa + kABytes;
          if (rank == 0) mbar_arrive_expect_tx(bar_full + 8 * slot, 2 * kPairStageBytes);
          tma_load_2d_pair(sa, &a_map, bar_full + 8 * slot, kb * kBlockK, tile.row0);
          const int bx = p.tiled ? 0 : kb * kBlockK, by = p.tiled ? kb * 128 : 0;
          tma_load_2d_pair(sb, &b_map, bar_full + 8 * slot, bx, b_row + by);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA ------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_f8(2 * kTileM, kTileN);
      const uint32_t peer_empty = mapa_u32(bar_empty, 1), peer_tfull = mapa_u32(bar_tfull, 1);
      uint32_t it = 0;
      bool alive = true;
      for (int w = pair_id; w < total && alive; w += n_pair_ctas) {
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t slot = it % kPairStages, phase = (it / kPairStages) & 1;
          const uint32_t buf = it & 1, aphase = (it >> 1) & 1;
          alive = mbar_wait(bar_full + 8 * slot, phase, p.err);
          alive = alive && mbar_wait(bar_tempty + 8 * buf, aphase ^ 1, p.err);
          if (!alive) break;
          tc_fence_after();
          const uint32_t sa = ring + slot * kPairStageBytes, sb = sa + kABytes;
          const uint64_t a_desc = umma_desc_k128(sa), b_desc = umma_desc_k128(sb);
          const uint32_t d = tmem_base + buf * kTileN;
#pragma unroll
          for (int k = 0; k < kBlockK / 32; ++k)
            tc_mma_f8_pair(d, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
          tc_commit_pair(bar_empty + 8 * slot);
          tc_commit_pair(peer_empty + 8 * slot);
          tc_commit_pair(bar_tfull + 8 * buf);
          tc_commit_pair(peer_tfull + 8 * buf);
        }
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ------------------------------------------- promotion + epilogue ------
    const int quarter = warp & 3;
    PromoCtx ctx;
    ctx.bar_tfull = bar_tfull;
    ctx.bar_tempty = mapa_u32(bar_tempty, 0);  // the issuer's barriers, from either CTA
    ctx.bar_amax = bar_amax;
    ctx.amax_sm = amax_sm;
    ctx.lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    ctx.half = (warp - 4) >> 2;
    ctx.r = quarter * 32 + lane;
    ctx.lane = lane;
    uint32_t it = 0, tile_it = 0;
    bool alive = true;
    for (int w = pair_id; w < total && alive; w += n_pair_ctas, ++tile_it) {
      const MoeTile tile = my_tile(w);
      alive = promo_tile<MODE, true>(p, ctx, tile, w % p.n_tiles, it, tile_it);
    }
  }

  // nobody leaves while the other CTA may still signal its barriers or read its shared memory
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
#endif
}

template <int MODE>
static int launch_pair(const CUtensorMap& a_map, const CUtensorMap& b_map, const GemmParams& p, cudaStream_t st) {
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  static bool attr_done[64] = {false};
  static int sm_count[64] = {0};
  if (dev < 64 && !attr_done[dev]) {
    B200_CUDA(cudaFuncSetAttribute(moe_fp8_gemm_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kPairSmem));
    B200_CUDA(cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
    attr_done[dev] = true;
  }
  const int sms = dev < 64 && sm_count[dev] > 0 ? sm_count[dev] : 148;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sms & ~1);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kPairSmem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B200_CUDA(cudaLaunchKernelEx(&cfg, moe_fp8_gemm_pair_kernel<MODE>, a_map, b_map, p));
  return 0;
}

int launch_gemm_pair(int mode, const CUtensorMap& a_map, const CUtensorMap& b_map, const GemmParams& p,
                     cudaStream_t st) {
  return mode == kModeGateUp ? launch_pair<kModeGateUp>(a_map, b_map, p, st)
                             : launch_pair<kModeDown>(a_map, b_map, p, st);
}

int gemm_pair_max_tiles() { return kPairMaxPairs; }

}  // namespace b200
