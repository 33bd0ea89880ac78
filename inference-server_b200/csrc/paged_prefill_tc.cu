// Tiled causal attention over KV pages for a chunk of prompt tokens on the tcgen05 tensor cores (sm_100a),
// head_dim 128 with 8 or 16 query heads per kv head.  Same operation, arguments and row order as
// paged_attn_prefill_kernel (paged_prefill.cu), which stays for the other head shapes; what it replaces in the
// reference is described there (src/inference_server/kv_cache/hf_format.py:21-45 gather +
// src/inference_server/backends/torch_backend.py:107-147 chunk forward).
//
//   grid     (query tiles, kv heads).  A CTA owns 128 rows of the score matrix: 128 / G consecutive prompt
//            positions x the G query heads of its kv head, and walks the key tiles (128 keys = 8 pages) of
//            the context up to its last position.  Heavy tiles (late positions) are issued first.
//   warp 0   TMA producer: the Q tile once (boxes of G rows x 128 B), then per key tile the 8 K pages and
//            the 8 V pages of the kv head (boxes of 16 tokens x 128 B, two column halves each) into two
//            two-stage rings, 128-byte swizzle, mbarrier hand-over.  The 16 boxes of a tile are issued by 16
//            lanes side by side.
//   warp 1   score issuer (one thread): S = Q K^T as 8 x tcgen05.mma M128 N128 K16 (kind::f16, bf16, both
//            operands K-major) into one of two S accumulators in TMEM, as far ahead as those allow.
//   warp 2   P V issuer (one thread): O += P V as 2 x 4 tcgen05.mma M128 N128 K16, P (bf16, written by the
//            softmax warps) as the K-major A operand and V as an MN-major B operand straight from its page
//            layout [key][head_dim].  A thread gets a tcgen05.mma on its way about every 95 cycles whatever
//            its N (measured), which is why the two products have an issuer each, and the P tile is handed
//            over in two halves of 64 keys so that the first half's product starts while the second half's
//            exponentials are still being taken.
//   warps 3-10  softmax: a thread owns one score row and 64 of the tile's 128 key columns (two threads per
//            row; TMEM lanes are bound to warp_id % 4, so warps w and w+4 of these see the same rows and
//            meet on a 64-thread named barrier).  tcgen05.ld of its half row, causal mask by position, row
//            max exchanged with the partner through shared memory, p = exp2((s - m) * scale) in fp32, P
//            stored as bf16 into its half of the swizzled A-operand tile once the product that read that
//            half for the tile before has finished.  The running max is lazy: O (in TMEM) and the running
//            sum are rescaled only when a row's max grew by more than 2^8 since the last rescale (any row
//            of the warp: the whole warp rescales, through tcgen05.ld / tcgen05.st, after both products of
//            the tile before have finished); until then p is taken against the older max, which is exact
//            after the final division by the sum taken against the same max.
//   out      O / l as bf16, each thread 128 contiguous bytes of its row.
//
// TMEM: S0 columns 0-127, S1 128-255, O 256-383 (512 allocated).  Shared memory: Q 32 KiB, P 32 KiB,
// K ring 2 x 32 KiB, V ring 2 x 32 KiB.  Every mbarrier wait is bounded; a wait that runs out records
// kErrDevWaitTimeout and the thread stops waiting but keeps the loop structure (the named barriers between
// partner warps are still met), so the kernel ends.

#include "common.cuh"
#include "host.h"

namespace b200 {

constexpr int kTcPage = 16;
constexpr int kTcRows = 128;                 // score rows per CTA = M of the MMAs
constexpr int kTcKeys = 128;                 // keys per tile = N of S, K of P V
constexpr int kTcPages = kTcKeys / kTcPage;
constexpr int kTcD = 128;
constexpr int kTcHalfBytes = 128 * 128;      // 128 rows x 64 bf16: one swizzled column half of a tile
constexpr int kTcTileBytes = 2 * kTcHalfBytes;
constexpr int kTcSoftmaxWarps = 8;
constexpr int kTcThreads = (3 + kTcSoftmaxWarps) * 32;
constexpr int kTcSmemTiles = 6;              // Q, P, K0, K1, V0, V1
constexpr int kTcExtraBytes = 256 /* barriers, tmem base */ + 2 * 2 * kTcRows * 4 /* max exchange */ +
                              2 * kTcRows * 4 /* sum exchange */;
constexpr int kTcSmemBytes = kTcSmemTiles * kTcTileBytes + 1024 + kTcExtraBytes;
constexpr float kTcRescaleLog2 = 8.f;        // rescale O when the max grew by more than this (log2 domain)

// bf16 x bf16 -> f32; A K-major; B K-major or (b_mn) MN-major.
__host__ __device__ constexpr uint32_t tc_idesc_bf16(uint32_t m, uint32_t n, uint32_t b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Descriptor of an MN-major operand tile with 128-byte swizzle: 64 elements of the M/N dimension are contiguous
// (128 B), consecutive K rows are 128 B apart, groups of 8 K rows `sbo` bytes apart, and the next 64 elements of
// the M/N dimension start `lbo` bytes further.
__device__ __forceinline__ uint64_t umma_desc_mn128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;  // 128-byte swizzle
  return d;
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
        "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The two warps that own the same 32 score rows (warp w and w + 4 of the softmax warps) meet here.
__device__ __forceinline__ void pair_barrier(int quarter) {
  switch (quarter) {
    case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
    case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
    default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
  }
}

// G: query heads per kv head (8 or 16).
template <int G>
__global__ void __launch_bounds__(kTcThreads, 1)
paged_attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                             const __grid_constant__ CUtensorMap v_map, const int* __restrict__ table_row,
                             __nv_bfloat16* __restrict__ out, int* __restrict__ err, int num_tokens, int first_pos,
                             int num_q_heads, int num_kv_heads, int num_blocks, float scale_log2) {
#ifdef B200_DEVICE_OK
  constexpr int QT = kTcRows / G;  // prompt positions per CTA
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_sm = base, p_sm = base + kTcTileBytes;
  const uint32_t k_sm = base + 2 * kTcTileBytes, v_sm = base + 4 * kTcTileBytes;  // two stages each
  const uint32_t bars = base + kTcSmemTiles * kTcTileBytes;
  const uint32_t bar_q = bars;                                   // Q tile landed
  const uint32_t bar_kfull = bars + 8, bar_kempty = bars + 24;   // [2] each
  const uint32_t bar_vfull = bars + 40, bar_vempty = bars + 56;  // [2] each
  const uint32_t bar_sfull = bars + 72, bar_sempty = bars + 88;  // [2] each: S accumulator written / read
  const uint32_t bar_pfull = bars + 104;                         // [2] a 64-key half of the P tile written
  const uint32_t bar_odone = bars + 120;                         // [2] the product over that half finished
  // [2, by tile parity] every softmax warp is past its rescale of O.  Two of them because a warp that needs no
  // rescale can get here for tile j + 1 before a warp of another quarter has arrived for tile j; it cannot get
  // to tile j + 2 before that (its P half waits for the product of tile j, which waits for this barrier).
  const uint32_t bar_rescaled = bars + 136;
  uint8_t* extra = base_ptr + kTcSmemTiles * kTcTileBytes;
  uint32_t* tmem_base_sm = reinterpret_cast<uint32_t*>(extra + 192);
  float* mx_sm = reinterpret_cast<float*>(extra + 256);          // [2 tiles][2 halves][128 rows]
  float* l_sm = mx_sm + 2 * 2 * kTcRows;                         // [2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 32) {
    tma_prefetch_desc(&q_map);
    tma_prefetch_desc(&k_map);
    tma_prefetch_desc(&v_map);
  }
  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_kempty + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_vempty + 8 * s, 1);
      mbar_init(bar_sfull + 8 * s, 1);
      mbar_init(bar_sempty + 8 * s, kTcSoftmaxWarps);
      mbar_init(bar_pfull + 8 * s, kTcSoftmaxWarps / 2);
      mbar_init(bar_odone + 8 * s, 1);
    }
    mbar_init(bar_rescaled, kTcSoftmaxWarps);
    mbar_init(bar_rescaled + 8, kTcSoftmaxWarps);
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_base_sm), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_sm;
  // Set-up done; Q and this chunk's K/V rows come from the kernel before this one.
  grid_dep_wait();
  grid_dep_launch();

  const int qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // late positions first
  const int h = blockIdx.y;
  const int t0 = qt * QT;
  const int t_end = min(t0 + QT, num_tokens);       // one past the tile's last real prompt token
  const int last_pos = first_pos + t_end - 1;       // last position any row of this CTA sees
  const int n_tiles = last_pos / kTcKeys + 1;
  const int last_page = last_pos / kTcPage;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA ------
    // Lanes 0-15 each own one box of a tile: page lane >> 1, column half lane & 1.
    if (lane == 0) mbar_arrive_expect_tx(bar_q, kTcTileBytes);
    __syncwarp();
    for (int i = lane; i < 2 * QT; i += 32) {
      const int tl = i >> 1, hf = i & 1;
      tma_load_2d(q_sm + hf * kTcHalfBytes + tl * G * 128, &q_map, bar_q, hf * 64,
                  (t0 + tl) * num_q_heads + h * G);  // rows past the chunk are filled with zeros
    }
    const int pg = (lane >> 1) & 7, hf = lane & 1;
    bool alive = true;
#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      // pages past the tile's last position hold nothing this CTA may read; the last valid page stands in so that
      // every stage is the same number of bytes and holds finite numbers (their scores are masked)
      int page = __ldg(table_row + min(j * kTcPages + pg, last_page));
      if (page < 0 || page >= num_blocks) {
        set_error(err, kErrDevBadBlockId);
        page = 0;
      }
      const int row = (page * num_kv_heads + h) * kTcPage;
      const uint32_t dst = st * kTcTileBytes + hf * kTcHalfBytes + pg * (kTcPage * 128);
      if (alive) alive = mbar_wait(bar_kempty + 8 * st, ph ^ 1, err);
      if (!__all_sync(0xffffffffu, alive)) break;
      if (lane == 0) mbar_arrive_expect_tx(bar_kfull + 8 * st, kTcTileBytes);
      __syncwarp();
      if (lane < 16) tma_load_2d(k_sm + dst, &k_map, bar_kfull + 8 * st, hf * 64, row);
      if (alive) alive = mbar_wait(bar_vempty + 8 * st, ph ^ 1, err);
      if (!__all_sync(0xffffffffu, alive)) break;
      if (lane == 0) mbar_arrive_expect_tx(bar_vfull + 8 * st, kTcTileBytes);
      __syncwarp();
      if (lane < 16) tma_load_2d(v_sm + dst, &v_map, bar_vfull + 8 * st, hf * 64, row);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------- S = Q K^T ------
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc_idesc_bf16(kTcRows, kTcKeys, 0);  // B = K, K-major
      bool alive = mbar_wait(bar_q, 0, err);
      const uint64_t a0 = umma_desc_k128(q_sm);
#pragma unroll 1
      for (int t = 0; t < n_tiles && alive; ++t) {
        const int st = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        alive = mbar_wait(bar_kfull + 8 * st, ph, err);
        if (!alive) break;
        alive = mbar_wait(bar_sempty + 8 * st, ph ^ 1, err);  // the softmax warps have read tile t - 2
        if (!alive) break;
        tc_fence_after();
        const uint64_t b0 = umma_desc_k128(k_sm + st * kTcTileBytes);
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // 16 of the 128 head dimensions each
          const uint32_t off = ((k >> 2) * kTcHalfBytes + (k & 3) * 32) >> 4;
          tc_mma_f16(tmem_base + st * kTcKeys, a0 + off, b0 + off, idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(bar_sfull + 8 * st);
        tc_commit(bar_kempty + 8 * st);
      }
    }
  } else if (warp == 2) {
    // ---------------------------------------------------- O += P V ------
    if (lane == 0) {
      constexpr uint32_t idesc_o = tc_idesc_bf16(kTcRows, kTcD, 1);  // B = V, MN-major
      const uint32_t tmem_o = tmem_base + 2 * kTcKeys;
      bool alive = true;
#pragma unroll 1
      for (int j = 0; j < n_tiles && alive; ++j) {
        const int st = j & 1;
        alive = mbar_wait(bar_vfull + 8 * st, (j >> 1) & 1, err);
        if (!alive) break;
        alive = mbar_wait(bar_rescaled + 8 * (j & 1), (j >> 1) & 1, err);  // nobody is rewriting O any more
        if (!alive) break;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          alive = mbar_wait(bar_pfull + 8 * half, j & 1, err);
          if (!alive) break;
          tc_fence_after();
          const uint64_t a0 = umma_desc_k128(p_sm + half * kTcHalfBytes);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {  // 16 keys each
            const uint64_t b = umma_desc_mn128(v_sm + st * kTcTileBytes + (half * 4 + kk) * (16 * 128), kTcHalfBytes, 1024);
            tc_mma_f16(tmem_o, a0 + ((kk * 32) >> 4), b, idesc_o, (j > 0 || half > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(bar_odone + 8 * half);
        }
        if (!alive) break;
        tc_commit(bar_vempty + 8 * st);
      }
    }
  } else {
    // -------------------------------------------------------- softmax ------
    const int sw = warp - 3;                 // 0..7
    const int hf = sw >> 2;                  // which 64 of the tile's 128 key columns (and of O's 128 columns)
    const int quarter = warp & 3;            // TMEM lanes this warp may touch
    const int r = quarter * 32 + lane;       // score row
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t tmem_o = lane_addr + 2 * kTcKeys + hf * 64;
    const int tl = r / G;
    const bool real = t0 + tl < num_tokens;
    const int pos = first_pos + min(t0 + tl, t_end - 1);  // the last key this row may see
    uint8_t* p_half = base_ptr + kTcTileBytes + hf * kTcHalfBytes;
    float m_run = -INFINITY, l_run = 0.f;
    bool alive = true;
#pragma unroll 1
    for (int j = 0; j < n_tiles; ++j) {
      const int buf = j & 1;
      if (alive) alive = mbar_wait(bar_sfull + 8 * buf, (j >> 1) & 1, err);
      tc_fence_after();
      uint32_t raw[64];
      {
        uint32_t (&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(raw);
        uint32_t (&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(raw + 32);
        tmem_ld32(lane_addr + buf * kTcKeys + hf * 64, lo);
        tmem_ld32(lane_addr + buf * kTcKeys + hf * 64 + 32, hi);
        tmem_ld_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sempty + 8 * buf);  // this S accumulator may be overwritten
      float s[64];
      const int kbase = j * kTcKeys + hf * 64;
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (kbase + 63 > pos) {  // the causal edge runs through this half row
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          s[c] = kbase + c > pos ? -INFINITY : __uint_as_float(raw[c]);
          mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          s[c] = __uint_as_float(raw[c]);
          mx4[c & 3] = fmaxf(mx4[c & 3], s[c]);
        }
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      float* mxb = mx_sm + buf * 2 * kTcRows;
      mxb[hf * kTcRows + r] = mx;
      pair_barrier(quarter);
      const float m_new = fmaxf(m_run, fmaxf(mx, mxb[(hf ^ 1) * kTcRows + r]));
      const bool need = (m_new - m_run) * scale_log2 > kTcRescaleLog2;  // true on the first tile (m_run = -inf)
      if (__any_sync(0xffffffffu, need)) {
        if (j > 0) {
          // O may be touched once both products of the tile before have finished
          if (alive) alive = mbar_wait(bar_odone + 8 * (hf ^ 1), (j - 1) & 1, err);
          if (alive) alive = mbar_wait(bar_odone + 8 * hf, (j - 1) & 1, err);
          const float alpha = fast_exp2((m_run - m_new) * scale_log2);
          l_run *= alpha;
          tc_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < 64; c0 += 32) {
            uint32_t o[32];
            tmem_ld32(tmem_o + c0, o);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
            tmem_st32(tmem_o + c0, o);
          }
          tmem_st_wait();
        }
        m_run = m_new;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_rescaled + 8 * buf);
      // this half of the P tile was last read by the product of the tile before
      if (j > 0 && alive) alive = mbar_wait(bar_odone + 8 * hf, (j - 1) & 1, err);
      const float mb = m_run * scale_log2;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) p[i] = fast_exp2(fmaf(s[ch * 8 + i], scale_log2, -mb));
        sum4[ch & 3] += ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
        uint4 w;
        w.x = pack_bf16x2(p[0], p[1]);
        w.y = pack_bf16x2(p[2], p[3]);
        w.z = pack_bf16x2(p[4], p[5]);
        w.w = pack_bf16x2(p[6], p[7]);
        *reinterpret_cast<uint4*>(p_half + swz128(r, ch)) = w;
      }
      l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      fence_proxy_async();  // the tensor core reads P through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull + 8 * hf);
    }
    // ---- epilogue: O / l, once both products of the last tile have finished
    if (alive) alive = mbar_wait(bar_odone + 8 * (hf ^ 1), (n_tiles - 1) & 1, err);
    if (alive) alive = mbar_wait(bar_odone + 8 * hf, (n_tiles - 1) & 1, err);
    tc_fence_after();
    l_sm[hf * kTcRows + r] = l_run;
    pair_barrier(quarter);
    const float inv = 1.f / (l_run + l_sm[(hf ^ 1) * kTcRows + r]);
    __nv_bfloat16* orow = out + (static_cast<size_t>(t0 + tl) * num_q_heads + h * G + (r - tl * G)) * kTcD + hf * 64;
#pragma unroll
    for (int c0 = 0; c0 < 64; c0 += 32) {
      uint32_t o[32];
      tmem_ld32(tmem_o + c0, o);
      tmem_ld_wait();
      if (real && alive) {
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
          w.y = pack_bf16x2(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
          w.z = pack_bf16x2(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
          w.w = pack_bf16x2(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c0 + c) = w;
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

static int launch_prefill_tc_g(int group, const CUtensorMap& qmap, const CUtensorMap& kmap, const CUtensorMap& vmap,
                               const int* table_row, void* out, int* err, int num_tokens, int first_pos, int hq, int hkv,
                               int num_blocks, float scale, cudaStream_t st) {
  const float sl = scale * 1.4426950408889634f;
  const int qt = kTcRows / group;
  const dim3 grid((num_tokens + qt - 1) / qt, hkv);
  if (group == 8) {
    int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&paged_attn_prefill_tc_kernel<8>), kTcSmemBytes);
    if (rc) return rc;
    B200_CUDA(launch_overlapped(paged_attn_prefill_tc_kernel<8>, grid, dim3(kTcThreads), kTcSmemBytes, st, qmap, kmap,
                                vmap, table_row, static_cast<__nv_bfloat16*>(out), err, num_tokens, first_pos, hq, hkv,
                                num_blocks, sl));
  } else {
    int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(&paged_attn_prefill_tc_kernel<16>), kTcSmemBytes);
    if (rc) return rc;
    B200_CUDA(launch_overlapped(paged_attn_prefill_tc_kernel<16>, grid, dim3(kTcThreads), kTcSmemBytes, st, qmap, kmap,
                                vmap, table_row, static_cast<__nv_bfloat16*>(out), err, num_tokens, first_pos, hq, hkv,
                                num_blocks, sl));
  }
  return 0;
}

// The tcgen05 form of the prompt attention: head_dim 128, 8 or 16 query heads per kv head, q and out 16-byte
// aligned.  Arguments as launch_prefill in paged_prefill.cu, which has checked them.
int launch_prefill_tc(const void* q, const void* k_pool, const void* v_pool, const int* table_row, void* out, int* err,
                      int num_tokens, int first_pos, int hq, int hkv, int num_blocks, float scale, cudaStream_t st) {
  const int group = hq / hkv;
  CUtensorMap qmap, kmap, vmap;
  const uint64_t rows = static_cast<uint64_t>(num_blocks) * hkv * kTcPage;
  int rc = get_tensor_map_2d(k_pool, rows, kTcD, 2, kTcPage, 64, &kmap);
  if (rc) return rc;
  rc = get_tensor_map_2d(v_pool, rows, kTcD, 2, kTcPage, 64, &vmap);
  if (rc) return rc;
  rc = get_tensor_map_2d(q, static_cast<uint64_t>(num_tokens) * hq, kTcD, 2, group, 64, &qmap);
  if (rc) return rc;
  return launch_prefill_tc_g(group, qmap, kmap, vmap, table_row, out, err, num_tokens, first_pos, hq, hkv, num_blocks,
                             scale, st);
}

}  // namespace b200
