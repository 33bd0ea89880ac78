// MoE routing, token permutation, activation quantisation and weighted combine.
//
// Semantics follow the router and expert dispatch the reference reaches through
// its model forward (src/inference_server/backends/torch_backend.py:305-322 ->
// transformers Qwen3MoeTopKRouter / grouped experts forward):
//   route    probabilities = softmax(logits) in fp32; the K largest are taken,
//            value descending, equal values by lower expert id; weights are the
//            selected probabilities, renormalised to sum to 1 when `renorm`.
//            Selection compares the logits themselves (softmax is monotone), so
//            expert ids do not depend on how exp() rounds.  Rows at or beyond an
//            optional device-side row count get expert id -1 ("no expert") and
//            weight 0: the permutation leaves such pairs out and the combine adds
//            nothing for them (padding rows of a fixed-shape step).
//   permute  the T*K (token, slot) pairs, numbered token-major, are stably
//            sorted by expert id: rows of one expert are contiguous and keep
//            ascending pair order.
//   quant    one scale per token per 128 columns: s = amax / 448 (1 when the
//            group is all zero), q = e4m3(x / s), stored with s.
//   combine  out[t] = sum_k w[t,k] * y[row_of_pair[t,k]] in fp32, k ascending.
// All of it is integer/byte work bound by launch latency and HBM traffic; none
// of it touches the tensor cores.

#include "common.cuh"
#include "host.h"

namespace b200 {

constexpr int kRouteWarps = 4;
constexpr int kRouteMaxPerLane = 8;  // num_experts <= 256

__device__ __forceinline__ float logit_f32(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float logit_f32(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

template <typename LT>
__global__ void __launch_bounds__(kRouteWarps * 32)
moe_route_kernel(const LT* __restrict__ logits, int T, int E, int K, int renorm,
                 const int* __restrict__ num_valid, int* __restrict__ topk_ids, float* __restrict__ topk_w) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  if (t >= T) return;
  if (num_valid != nullptr && t >= *num_valid) {
    if (lane < K) {
      topk_ids[static_cast<size_t>(t) * K + lane] = -1;
      topk_w[static_cast<size_t>(t) * K + lane] = 0.f;
    }
    return;
  }
  float v[kRouteMaxPerLane];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kRouteMaxPerLane; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < E ? logit_f32(logits, static_cast<size_t>(t) * E + e) : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float den = 0.f;
#pragma unroll
  for (int j = 0; j < kRouteMaxPerLane; ++j)
    if (lane + 32 * j < E) den += expf(v[j] - mx);
  den = warp_sum(den);

  unsigned taken = 0;  // bit j: this lane's candidate j has been selected
  float sel_sum = 0.f, my_p = 0.f;
  int my_id = 0;
  for (int k = 0; k < K; ++k) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kRouteMaxPerLane; ++j) {
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
    const float p = expf(bv - mx);
    sel_sum += p;
    if (lane == k) {
      my_p = p;
      my_id = be;
    }
  }
  if (lane < K) {
    topk_ids[static_cast<size_t>(t) * K + lane] = my_id;
    topk_w[static_cast<size_t>(t) * K + lane] = my_p / (renorm ? sel_sum : den);
  }
}

// ---------------------------------------------------------------- permute ---
constexpr int kRankThreads = 256;

// One CTA per expert: stable rank of every pair routed to this expert.
__global__ void __launch_bounds__(kRankThreads)
moe_rank_kernel(const int* __restrict__ topk_ids, int n_pairs, int* __restrict__ rank,
                int* __restrict__ counts) {
  __shared__ int warp_tot[kRankThreads / 32];
  grid_dep_wait();
  grid_dep_launch();
  const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = (n_pairs + kRankThreads - 1) / kRankThreads;
  const int lo = min(n_pairs, tid * chunk), hi = min(n_pairs, lo + chunk);
  // Latency-bound (a few KiB of ids per CTA): a thread's ids are read once, eight at a time into registers
  // (all loads of a group in flight together), and the prefix over the threads is one shuffle scan plus one
  // exchange of eight warp totals instead of a scan through shared memory.
  constexpr int kHold = 16;
  int held[kHold];
  int c = 0;
#pragma unroll
  for (int u = 0; u < kHold; ++u) held[u] = lo + u < hi ? topk_ids[lo + u] : -2;
#pragma unroll
  for (int u = 0; u < kHold; ++u) c += held[u] == e;
  for (int i = lo + kHold; i < hi; ++i) c += topk_ids[i] == e;
  int inc = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += y;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  int before = 0, total = 0;
#pragma unroll
  for (int w = 0; w < kRankThreads / 32; ++w) {
    const int t = warp_tot[w];
    if (w < warp) before += t;
    total += t;
  }
  int run = before + inc - c;  // exclusive prefix: pairs of this expert in the threads before this one
#pragma unroll
  for (int u = 0; u < kHold; ++u)
    if (held[u] == e) rank[lo + u] = run++;
  for (int i = lo + kHold; i < hi; ++i)
    if (topk_ids[i] == e) rank[i] = run++;
  if (tid == 0) counts[e] = total;
}

constexpr int kScatterThreads = 256;

__global__ void __launch_bounds__(kScatterThreads)
moe_scatter_kernel(const int* __restrict__ topk_ids, const int* __restrict__ rank,
                   const int* __restrict__ counts, int n_pairs, int E, int tile_experts, int tile_rows,
                   int* __restrict__ sorted_pair, int* __restrict__ row_of_pair,
                   int* __restrict__ expert_offsets, MoeTile* __restrict__ tiles,
                   int* __restrict__ num_tiles, int* __restrict__ err) {
  extern __shared__ int sm[];  // counts[E], offsets[E + 1]
  int* cnt = sm;
  int* off = sm + E;
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += kScatterThreads) cnt[e] = counts[e];
  __syncthreads();
  for (int e = tid; e <= E; e += kScatterThreads) {
    int s = 0;
    for (int j = 0; j < e; ++j) s += cnt[j];
    off[e] = s;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int e = tid; e <= E; e += kScatterThreads) expert_offsets[e] = off[e];
    if (tiles != nullptr) {
      // only the first `tile_experts` experts get row tiles (a trailing dummy expert that collects empty
      // slots is sorted but never multiplied)
      for (int e = tid; e < tile_experts; e += kScatterThreads) {
        int tp = 0;
        for (int j = 0; j < e; ++j) tp += (cnt[j] + tile_rows - 1) / tile_rows;
        const int nt = (cnt[e] + tile_rows - 1) / tile_rows;
        for (int j = 0; j < nt; ++j) {
          MoeTile t;
          t.expert = e;
          t.row0 = off[e] + j * tile_rows;
          t.rows = min(tile_rows, cnt[e] - j * tile_rows);
          t.pad = 0;
          tiles[tp + j] = t;
        }
        if (e == tile_experts - 1) *num_tiles = tp + nt;
      }
    }
  }
  const int i = blockIdx.x * kScatterThreads + tid;
  if (i < n_pairs) {
    const int e = topk_ids[i];
    if (e < 0 || e >= E) {
      if (e != -1) set_error(err, kErrDevBadExpert);  // -1 is "no expert": the pair is left out, not an error
      row_of_pair[i] = -1;
    } else {
      const int dst = off[e] + rank[i];
      sorted_pair[dst] = i;
      row_of_pair[i] = dst;
    }
  }
}

// moe_scatter_kernel fused with the row copy that follows it on the receive side of the expert-parallel
// exchange: one CTA per received slot computes the slot's sorted position and copies its e4m3 row and scales
// there.  Slots of experts >= tile_experts (the dummy expert that collects empty slots) are ranked, not copied.
__global__ void __launch_bounds__(256)
moe_scatter_rows_kernel(const int* __restrict__ ids, const int* __restrict__ rank,
                        const int* __restrict__ counts, int E, int tile_experts, int H, int tile_rows,
                        int* __restrict__ sorted_pair, int* __restrict__ row_of_pair,
                        int* __restrict__ expert_offsets, MoeTile* __restrict__ tiles,
                        int* __restrict__ num_tiles, const uint8_t* __restrict__ src_q,
                        const float* __restrict__ src_s, uint8_t* __restrict__ dst_q,
                        float* __restrict__ dst_s, int* __restrict__ err) {
  extern __shared__ int sm[];  // counts[E], offsets[E + 1]
  int* cnt = sm;
  int* off = sm + E;
  const int tid = threadIdx.x, nthr = blockDim.x;
  // Latency-bound: the slot's expert, its rank and the first pieces of its row and scales are asked for before
  // the counts are summed; where they go is known only afterwards.
  const int i = blockIdx.x;
  const int e = ids[i];
  const int slot_rank = rank[i];
  const int groups = H / 128;
  const uint4* s4 = reinterpret_cast<const uint4*>(src_q + static_cast<size_t>(i) * H);
  const bool live = e >= 0 && e < tile_experts;  // a slot whose row is copied
  uint4 first_piece = make_uint4(0u, 0u, 0u, 0u);
  float first_scale = 0.f;
  if (live && tid < H / 16) first_piece = s4[tid];
  if (live && tid < groups) first_scale = src_s[static_cast<size_t>(i) * groups + tid];
  for (int e2 = tid; e2 < E; e2 += nthr) cnt[e2] = counts[e2];
  __syncthreads();
  for (int e2 = tid; e2 <= E; e2 += nthr) {
    int s = 0;
    for (int j = 0; j < e2; ++j) s += cnt[j];
    off[e2] = s;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int e2 = tid; e2 <= E; e2 += nthr) expert_offsets[e2] = off[e2];
    for (int e2 = tid; e2 < tile_experts; e2 += nthr) {
      int tp = 0;
      for (int j = 0; j < e2; ++j) tp += (cnt[j] + tile_rows - 1) / tile_rows;
      const int nt = (cnt[e2] + tile_rows - 1) / tile_rows;
      for (int j = 0; j < nt; ++j) {
        MoeTile t;
        t.expert = e2;
        t.row0 = off[e2] + j * tile_rows;
        t.rows = min(tile_rows, cnt[e2] - j * tile_rows);
        t.pad = 0;
        tiles[tp + j] = t;
      }
      if (e2 == tile_experts - 1) *num_tiles = tp + nt;
    }
  }
  if (e < 0 || e >= E) {
    if (tid == 0) set_error(err, kErrDevBadExpert);
    return;
  }
  const int dst = off[e] + slot_rank;
  if (tid == 0) {
    sorted_pair[dst] = i;
    row_of_pair[i] = dst;
  }
  if (e >= tile_experts) return;
  uint4* d4 = reinterpret_cast<uint4*>(dst_q + static_cast<size_t>(dst) * H);
  if (tid < H / 16) d4[tid] = first_piece;
  for (int c = tid + nthr; c < H / 16; c += nthr) d4[c] = s4[c];
  if (tid < groups) dst_s[static_cast<size_t>(dst) * groups + tid] = first_scale;
  for (int gidx = tid + nthr; gidx < groups; gidx += nthr)
    dst_s[static_cast<size_t>(dst) * groups + gidx] = src_s[static_cast<size_t>(i) * groups + gidx];
}

// ------------------------------------------------------ activation quant ----
// One CTA per token, 8 columns per thread.  When row_of_pair is given the
// quantised row is written to each of the token's K sorted rows; otherwise to
// row t.
__global__ void act_quant_scatter_kernel(const __nv_bfloat16* __restrict__ x,
                                         const int* __restrict__ row_of_pair, int H, int K,
                                         uint8_t* __restrict__ xq, float* __restrict__ xs) {
  const int t = blockIdx.x, tid = threadIdx.x;
  const uint4 raw = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H + tid * 8);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float f[8];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 p = __bfloat1622float2(h2[j]);
    f[2 * j] = p.x;
    f[2 * j + 1] = p.y;
    amax = fmaxf(amax, fmaxf(fabsf(p.x), fabsf(p.y)));
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = amax > 0.f ? amax / 448.f : 1.f;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    lo |= static_cast<uint32_t>(to_e4m3(f[j] / s)) << (8 * j);
    hi |= static_cast<uint32_t>(to_e4m3(f[4 + j] / s)) << (8 * j);
  }
  const int groups = H / 128;
  const int reps = row_of_pair ? K : 1;
  for (int k = 0; k < reps; ++k) {
    const int row = row_of_pair ? row_of_pair[static_cast<size_t>(t) * K + k] : t;
    *reinterpret_cast<uint2*>(xq + static_cast<size_t>(row) * H + tid * 8) = make_uint2(lo, hi);
    if ((tid & 15) == 0) xs[static_cast<size_t>(row) * groups + (tid >> 4)] = s;
  }
}

// Exclusive prefix sums of v[0..n) into out[0..n] (out[n] = total); n <= 1024, all threads call.
__device__ __forceinline__ void block_exclusive_scan(const int* v, int* out, int n, int* warp_tot) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nthreads = blockDim.x;
  int carry = 0;
  for (int base = 0; base < n; base += nthreads) {
    const int i = base + tid;
    const int x = i < n ? v[i] : 0;
    int inc = x;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += y;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    int woff = 0, total = 0;
    for (int w = 0; w < (nthreads + 31) / 32; ++w) {
      const int t = warp_tot[w];
      if (w < warp) woff += t;
      total += t;
    }
    if (i < n) out[i] = carry + woff + inc - x;
    carry += total;
    __syncthreads();
  }
  if (tid == 0) out[n] = carry;
  __syncthreads();
}

// Scatter + activation quantisation in one pass.  One CTA per token, 8 columns per
// thread: every CTA rebuilds the expert offsets from the counts (a 128-entry scan),
// places the token's K pairs, quantises the token row once and writes it to its K
// sorted rows.  CTA 0 also publishes the offsets and the row tiles.
__global__ void moe_scatter_quant_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ topk_ids,
                                         const int* __restrict__ rank, const int* __restrict__ counts,
                                         int E, int K, int H, int tile_rows, int* __restrict__ sorted_pair,
                                         int* __restrict__ row_of_pair, int* __restrict__ expert_offsets,
                                         MoeTile* __restrict__ tiles, int* __restrict__ num_tiles,
                                         uint8_t* __restrict__ xq, float* __restrict__ xs,
                                         int* __restrict__ err, int ep_world, int ep_capacity,
                                         int* __restrict__ slot_of_pair, int* __restrict__ expert_of_slot,
                                         int* __restrict__ overflow, const EpPeers peers) {
  extern __shared__ int sm[];  // cnt[E], off[E+1], ntile[E], toff[E+1], warp_tot[32], dst[K]
  grid_dep_wait();
  grid_dep_launch();
  const bool p2p = peers.xq[0] != nullptr;
  int* cnt = sm;
  int* off = cnt + E;
  int* ntile = off + E + 1;
  int* toff = ntile + E;
  int* warp_tot = toff + E + 1;
  int* dst = warp_tot + 32;
  const int t = blockIdx.x, tid = threadIdx.x;
  // Latency-bound: the token's row and (threads < K) its pair's expert and rank are asked for first, so that they
  // travel while the counts are scanned.
  const uint4 raw = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H + tid * 8);
  int my_e = -1, pair_rank = 0;
  if (tid < K) {
    my_e = topk_ids[t * K + tid];
    pair_rank = rank[t * K + tid];
  }
  for (int e = tid; e < E; e += blockDim.x) {
    cnt[e] = counts[e];
    ntile[e] = (cnt[e] + tile_rows - 1) / tile_rows;
  }
  __syncthreads();
  block_exclusive_scan(cnt, off, E, warp_tot);
  if (t == 0) {
    block_exclusive_scan(ntile, toff, E, warp_tot);
    for (int e = tid; e <= E; e += blockDim.x) expert_offsets[e] = off[e];
    for (int e = tid; e < E; e += blockDim.x)
      for (int j = 0; j < ntile[e]; ++j) {
        MoeTile tl;
        tl.expert = e;
        tl.row0 = off[e] + j * tile_rows;
        tl.rows = min(tile_rows, cnt[e] - j * tile_rows);
        tl.pad = 0;
        tiles[toff[e] + j] = tl;
      }
    if (tid == 0) *num_tiles = toff[E];
  }
  if (tid < K) {
    const int pair = t * K + tid;
    const int e = my_e;
    int d = -1;
    if (e < 0 || e >= E) {
      if (e != -1) set_error(err, kErrDevBadExpert);  // -1 is "no expert": the pair is left out, not an error
      row_of_pair[pair] = -1;
      if (slot_of_pair != nullptr) slot_of_pair[pair] = -1;
    } else {
      d = off[e] + pair_rank;
      sorted_pair[d] = pair;
      row_of_pair[pair] = d;
      if (slot_of_pair != nullptr) {
        // expert-parallel dispatch: the row goes to slot (position among this rank's rows for the owner of
        // expert e) of that owner's segment of the send buffer; rows past the capacity are dropped and flagged
        const int e_local = E / ep_world, owner = e / e_local;
        const int pos = d - off[owner * e_local];
        if (pos < ep_capacity) {
          d = owner * ep_capacity + pos;
          if (p2p) peers.id[owner][peers.my_rank * ep_capacity + pos] = e - owner * e_local;
          else expert_of_slot[d] = e - owner * e_local;
        } else {
          d = -1;
          *overflow = 1;
        }
        slot_of_pair[pair] = d;
      }
    }
    dst[tid] = d;
  }
  if (slot_of_pair != nullptr) {
    // slots past the rows a destination gets carry the dummy expert id E/W, which gets no tiles there
    const int e_local = E / ep_world, total = ep_world * ep_capacity;
    for (int i = t * blockDim.x + tid; i < total; i += gridDim.x * blockDim.x) {
      const int owner = i / ep_capacity, pos = i - owner * ep_capacity;
      if (pos >= off[(owner + 1) * e_local] - off[owner * e_local]) {
        if (p2p) peers.id[owner][peers.my_rank * ep_capacity + pos] = e_local;
        else expert_of_slot[i] = e_local;
      }
    }
  }
  __syncthreads();

  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float f[8];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 p = __bfloat1622float2(h2[j]);
    f[2 * j] = p.x;
    f[2 * j + 1] = p.y;
    amax = fmaxf(amax, fmaxf(fabsf(p.x), fabsf(p.y)));
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float s = amax > 0.f ? amax / 448.f : 1.f;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    lo |= static_cast<uint32_t>(to_e4m3(f[j] / s)) << (8 * j);
    hi |= static_cast<uint32_t>(to_e4m3(f[4 + j] / s)) << (8 * j);
  }
  const int groups = H / 128;
  for (int k = 0; k < K; ++k) {
    int row = dst[k];
    if (row < 0) continue;
    uint8_t* q = xq;
    float* sc = xs;
    if (p2p) {  // straight into the owner's receive buffers over NVLink (or this GPU's own, for its experts)
      const int owner = row / ep_capacity;
      row = peers.my_rank * ep_capacity + (row - owner * ep_capacity);
      q = peers.xq[owner];
      sc = peers.xs[owner];
    }
    *reinterpret_cast<uint2*>(q + static_cast<size_t>(row) * H + tid * 8) = make_uint2(lo, hi);
    if ((tid & 15) == 0) sc[static_cast<size_t>(row) * groups + (tid >> 4)] = s;
  }
}

// ------------------------------------------------------------- combine ------
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y,
                                   const int* __restrict__ row_of_pair,
                                   const float* __restrict__ topk_w, int H, int K,
                                   __nv_bfloat16* __restrict__ out) {
  const int t = blockIdx.x, tid = threadIdx.x;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < K; ++k) {
    const int row = row_of_pair[static_cast<size_t>(t) * K + k];
    if (row < 0) continue;  // a pair without a result row (dropped by the expert-parallel capacity) adds nothing
    const float w = topk_w[static_cast<size_t>(t) * K + k];
    const uint4 raw = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(row) * H + tid * 8);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 p = __bfloat1622float2(h2[j]);
      acc[2 * j] += w * p.x;
      acc[2 * j + 1] += w * p.y;
    }
  }
  uint4 o;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + tid * 8) = o;
}

// combine fused with the next block's residual add and RMSNorm:
//   delta = bf16(sum_k w * y);  x = bf16(x + delta);  out = weight * rmsnorm(x)
__global__ void moe_combine_add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ y,
                                               const int* __restrict__ row_of_pair,
                                               const float* __restrict__ topk_w, int H, int K,
                                               __nv_bfloat16* __restrict__ x,
                                               const __nv_bfloat16* __restrict__ weight, float eps,
                                               __nv_bfloat16* __restrict__ out) {
  __shared__ float red[32];
  grid_dep_wait();
  grid_dep_launch();
  const int t = blockIdx.x, tid = threadIdx.x;
  // The kernel is a chain of dependent loads (pair -> result row -> its values) on a few KiB per CTA, so it is
  // bound by memory latency: everything that does not depend on another load is asked for at once - the
  // residual row and the norm weights here, then up to eight row numbers, then those rows together.  The sums
  // are taken in pair order as before.
  const size_t base = static_cast<size_t>(t) * H + tid * 8;
  uint4 xr = *reinterpret_cast<const uint4*>(x + base);
  const uint4 wraw = *reinterpret_cast<const uint4*>(weight + tid * 8);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += 8) {
    int rows[8];
    float ws[8];
    uint4 raws[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const bool in = k0 + u < K;
      // a pair without a result row (dropped by the expert-parallel capacity) has row -1 and adds nothing
      rows[u] = in ? row_of_pair[static_cast<size_t>(t) * K + k0 + u] : -1;
      ws[u] = in ? topk_w[static_cast<size_t>(t) * K + k0 + u] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (rows[u] >= 0) raws[u] = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(rows[u]) * H + tid * 8);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (rows[u] < 0) continue;
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raws[u]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 p = __bfloat1622float2(h2[j]);
        acc[2 * j] += ws[u] * p.x;
        acc[2 * j + 1] += ws[u] * p.y;
      }
    }
  }
  __nv_bfloat162* x2 = reinterpret_cast<__nv_bfloat162*>(&xr);
  float f[8], ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    x2[j] = __hadd2(x2[j], __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]));
    const float2 p = __bfloat1622float2(x2[j]);
    f[2 * j] = p.x;
    f[2 * j + 1] = p.y;
    ss += p.x * p.x + p.y * p.y;
  }
  *reinterpret_cast<uint4*>(x + base) = xr;
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = (tid & 31) < (blockDim.x + 31) / 32 ? red[tid & 31] : 0.f;
  tot = warp_sum(tot);
  const float inv = rsqrtf(tot / static_cast<float>(H) + eps);
  const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wraw);
  uint4 o;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    o2[j] = __hmul2(w2[j], __floats2bfloat162_rn(f[2 * j] * inv, f[2 * j + 1] * inv));
  *reinterpret_cast<uint4*>(out + base) = o;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_route(const void* logits, int logits_dtype, int num_tokens, int num_experts,
                              int top_k, int renormalize, const int32_t* num_valid_rows, int32_t* topk_ids,
                              float* topk_weights, void* stream) {
  B200_REQUIRE(logits && topk_ids && topk_weights, "moe_route: null pointer");
  B200_REQUIRE(num_tokens >= 0, "moe_route: negative token count");
  B200_REQUIRE(logits_dtype == 0 || logits_dtype == 1, "moe_route: logits dtype %d is neither 0 (bf16) nor 1 (f32)",
               logits_dtype);
  B200_REQUIRE(num_experts > 0 && num_experts <= 32 * kRouteMaxPerLane,
               "moe_route: num_experts %d outside [1, %d]", num_experts, 32 * kRouteMaxPerLane);
  B200_REQUIRE(top_k > 0 && top_k <= 32 && top_k <= num_experts,
               "moe_route: top_k %d outside [1, min(32, num_experts)]", top_k);
  int rc = check_device(nullptr);
  if (rc) return rc;
  if (num_tokens == 0) return 0;
  const int blocks = (num_tokens + kRouteWarps - 1) / kRouteWarps;
  if (logits_dtype == 1)
    moe_route_kernel<float><<<blocks, kRouteWarps * 32, 0, as_stream(stream)>>>(
        static_cast<const float*>(logits), num_tokens, num_experts, top_k, renormalize, num_valid_rows, topk_ids,
        topk_weights);
  else
    moe_route_kernel<__nv_bfloat16><<<blocks, kRouteWarps * 32, 0, as_stream(stream)>>>(
        static_cast<const __nv_bfloat16*>(logits), num_tokens, num_experts, top_k, renormalize, num_valid_rows,
        topk_ids, topk_weights);
  B200_CUDA(cudaGetLastError());
  return 0;
}

// Workspace layout: [status word, 256 B][counts: E ints][rank: T*K ints]
extern "C" size_t b200_moe_permute_workspace_bytes(int num_tokens, int num_experts, int top_k) {
  if (num_tokens < 0 || num_experts <= 0 || top_k <= 0) return 256;
  size_t off = 256;
  off += (static_cast<size_t>(num_experts) * 4 + 255) & ~size_t(255);
  off += (static_cast<size_t>(num_tokens) * top_k * 4 + 255) & ~size_t(255);
  return off;
}

extern "C" int b200_moe_max_tiles(int num_tokens, int num_experts, int top_k) {
  if (num_tokens < 0 || num_experts <= 0 || top_k <= 0) return 0;
  return (num_tokens * top_k + 127) / 128 + num_experts;
}

extern "C" int b200_moe_permute(const int32_t* topk_ids, int num_tokens, int num_experts, int top_k,
                                int32_t* sorted_pair_ids, int32_t* row_of_pair,
                                int32_t* expert_offsets, void* tiles, int32_t* num_tiles,
                                int tile_experts, void* workspace, size_t workspace_bytes, void* stream) {
  B200_REQUIRE(topk_ids && sorted_pair_ids && row_of_pair && expert_offsets && workspace,
               "moe_permute: null pointer");
  B200_REQUIRE((tiles == nullptr) == (num_tiles == nullptr),
               "moe_permute: tiles and num_tiles must be given together");
  B200_REQUIRE(num_tokens >= 0 && num_experts > 0 && num_experts <= 1024 && top_k > 0,
               "moe_permute: bad dimensions T=%d E=%d K=%d", num_tokens, num_experts, top_k);
  B200_REQUIRE(tile_experts >= 0 && tile_experts <= num_experts, "moe_permute: tile_experts %d outside [0, %d]",
               tile_experts, num_experts);
  if (tile_experts == 0) tile_experts = num_experts;
  const size_t need = b200_moe_permute_workspace_bytes(num_tokens, num_experts, top_k);
  if (workspace_bytes < need) {
    set_detail("moe_permute: workspace %zu < required %zu", workspace_bytes, need);
    return -kErrWorkspace;
  }
  int rc = check_device(nullptr);
  if (rc) return rc;
  cudaStream_t st = as_stream(stream);
  uint8_t* p = static_cast<uint8_t*>(workspace);
  int* err = reinterpret_cast<int*>(p);
  int* counts = reinterpret_cast<int*>(p + 256);
  int* rank = reinterpret_cast<int*>(p + 256 + ((static_cast<size_t>(num_experts) * 4 + 255) & ~size_t(255)));
  const int n_pairs = num_tokens * top_k;
  moe_rank_kernel<<<num_experts, kRankThreads, 0, st>>>(topk_ids, n_pairs, rank, counts);
  B200_CUDA(cudaGetLastError());
  const int blocks = n_pairs > 0 ? (n_pairs + kScatterThreads - 1) / kScatterThreads : 1;
  moe_scatter_kernel<<<blocks, kScatterThreads, (2 * num_experts + 1) * sizeof(int), st>>>(
      topk_ids, rank, counts, n_pairs, num_experts, tile_experts, 128, sorted_pair_ids, row_of_pair,
      expert_offsets, static_cast<MoeTile*>(tiles), num_tiles, err);
  B200_CUDA(cudaGetLastError());
  return 0;
}

static int permute_quant_impl(const int32_t* topk_ids, const void* x, int num_tokens, int num_experts,
                              int top_k, int hidden, int32_t* sorted_pair_ids, int32_t* row_of_pair,
                              int32_t* expert_offsets, void* tiles, int32_t* num_tiles, void* xq,
                              float* x_scale, void* workspace, size_t workspace_bytes, int ep_world,
                              int ep_capacity, int32_t* slot_of_pair, int32_t* expert_of_slot,
                              int32_t* overflow, const EpPeers& peers, void* stream) {
  B200_REQUIRE(topk_ids && x && sorted_pair_ids && row_of_pair && expert_offsets && tiles && num_tiles && xq &&
                   x_scale && workspace,
               "moe_permute_quant: null pointer");
  B200_REQUIRE(num_tokens >= 0 && num_experts > 0 && num_experts <= 1024 && top_k > 0,
               "moe_permute_quant: bad dimensions T=%d E=%d K=%d", num_tokens, num_experts, top_k);
  B200_REQUIRE(hidden > 0 && hidden % 256 == 0 && hidden <= 8192 && top_k <= hidden / 8,
               "moe_permute_quant: hidden %d must be a multiple of 256, <= 8192 and >= 8 * top_k", hidden);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(xq) & 7) == 0,
               "moe_permute_quant: x must be 16-byte and xq 8-byte aligned");
  const size_t need = b200_moe_permute_workspace_bytes(num_tokens, num_experts, top_k);
  if (workspace_bytes < need) {
    set_detail("moe_permute_quant: workspace %zu < required %zu", workspace_bytes, need);
    return -kErrWorkspace;
  }
  int rc = check_device(nullptr);
  if (rc) return rc;
  cudaStream_t st = as_stream(stream);
  if (num_tokens == 0) {
    // nothing to place, but a GEMM that follows must not find the previous call's tiles
    B200_CUDA(cudaMemsetAsync(num_tiles, 0, sizeof(int32_t), st));
    B200_CUDA(cudaMemsetAsync(expert_offsets, 0, (static_cast<size_t>(num_experts) + 1) * sizeof(int32_t), st));
    return 0;
  }
  uint8_t* p = static_cast<uint8_t*>(workspace);
  int* err = reinterpret_cast<int*>(p);
  int* counts = reinterpret_cast<int*>(p + 256);
  int* rank = reinterpret_cast<int*>(p + 256 + ((static_cast<size_t>(num_experts) * 4 + 255) & ~size_t(255)));
  B200_CUDA(launch_overlapped(moe_rank_kernel, dim3(num_experts), dim3(kRankThreads), 0, st, topk_ids,
                              num_tokens * top_k, rank, counts));
  const size_t smem = (4 * static_cast<size_t>(num_experts) + 2 + 32 + top_k) * sizeof(int);
  B200_CUDA(launch_overlapped(moe_scatter_quant_kernel, dim3(num_tokens), dim3(hidden / 8), smem, st,
                              static_cast<const __nv_bfloat16*>(x), topk_ids, rank, counts, num_experts, top_k, hidden,
                              128, sorted_pair_ids, row_of_pair, expert_offsets, static_cast<MoeTile*>(tiles),
                              num_tiles, static_cast<uint8_t*>(xq), x_scale, err, ep_world, ep_capacity, slot_of_pair,
                              expert_of_slot, overflow, peers));
  return 0;
}

extern "C" int b200_moe_permute_quant(const int32_t* topk_ids, const void* x, int num_tokens,
                                      int num_experts, int top_k, int hidden, int32_t* sorted_pair_ids,
                                      int32_t* row_of_pair, int32_t* expert_offsets, void* tiles,
                                      int32_t* num_tiles, void* xq, float* x_scale, void* workspace,
                                      size_t workspace_bytes, void* stream) {
  return permute_quant_impl(topk_ids, x, num_tokens, num_experts, top_k, hidden, sorted_pair_ids, row_of_pair,
                            expert_offsets, tiles, num_tiles, xq, x_scale, workspace, workspace_bytes, 1, 0,
                            nullptr, nullptr, nullptr, EpPeers{}, stream);
}

extern "C" int b200_moe_permute_quant_ep(const int32_t* topk_ids, const void* x, int num_tokens,
                                         int num_experts, int top_k, int hidden, int ep_world,
                                         int ep_capacity, int32_t* sorted_pair_ids, int32_t* row_of_pair,
                                         int32_t* expert_offsets, void* tiles, int32_t* num_tiles,
                                         void* xq_send, float* x_scale_send, int32_t* slot_of_pair,
                                         int32_t* expert_of_slot, int32_t* overflow, void* workspace,
                                         size_t workspace_bytes, void* stream) {
  B200_REQUIRE(ep_world >= 1 && num_experts % ep_world == 0 && ep_capacity > 0,
               "moe_permute_quant_ep: %d experts over %d ranks, capacity %d", num_experts, ep_world, ep_capacity);
  B200_REQUIRE(slot_of_pair && expert_of_slot && overflow, "moe_permute_quant_ep: null pointer");
  return permute_quant_impl(topk_ids, x, num_tokens, num_experts, top_k, hidden, sorted_pair_ids, row_of_pair,
                            expert_offsets, tiles, num_tiles, xq_send, x_scale_send, workspace, workspace_bytes,
                            ep_world, ep_capacity, slot_of_pair, expert_of_slot, overflow, EpPeers{}, stream);
}

extern "C" int b200_moe_permute_quant_ep_p2p(const int32_t* topk_ids, const void* x, int num_tokens,
                                             int num_experts, int top_k, int hidden, int ep_world,
                                             int ep_capacity, int ep_rank, int32_t* sorted_pair_ids,
                                             int32_t* row_of_pair, int32_t* expert_offsets, void* tiles,
                                             int32_t* num_tiles, void* const* xq_peers, void* const* xs_peers,
                                             void* const* id_peers, int32_t* slot_of_pair, int32_t* overflow,
                                             void* workspace, size_t workspace_bytes, void* stream) {
  B200_REQUIRE(ep_world >= 1 && ep_world <= kMaxEpWorld && num_experts % ep_world == 0 && ep_capacity > 0 &&
                   ep_rank >= 0 && ep_rank < ep_world,
               "moe_permute_quant_ep_p2p: %d experts over %d ranks (at most %d), capacity %d, rank %d", num_experts,
               ep_world, kMaxEpWorld, ep_capacity, ep_rank);
  B200_REQUIRE(slot_of_pair && overflow && xq_peers && xs_peers && id_peers, "moe_permute_quant_ep_p2p: null pointer");
  EpPeers peers{};
  for (int r = 0; r < ep_world; ++r) {
    B200_REQUIRE(xq_peers[r] && xs_peers[r] && id_peers[r], "moe_permute_quant_ep_p2p: null buffer of rank %d", r);
    B200_REQUIRE((reinterpret_cast<uintptr_t>(xq_peers[r]) & 7) == 0,
                 "moe_permute_quant_ep_p2p: xq of rank %d is not 8-byte aligned", r);
    peers.xq[r] = static_cast<uint8_t*>(xq_peers[r]);
    peers.xs[r] = static_cast<float*>(xs_peers[r]);
    peers.id[r] = static_cast<int*>(id_peers[r]);
  }
  peers.my_rank = ep_rank;
  return permute_quant_impl(topk_ids, x, num_tokens, num_experts, top_k, hidden, sorted_pair_ids, row_of_pair,
                            expert_offsets, tiles, num_tiles, peers.xq[ep_rank], peers.xs[ep_rank], workspace,
                            workspace_bytes, ep_world, ep_capacity, slot_of_pair, nullptr, overflow, peers, stream);
}

// Copies quantised rows and their scales into a new row order: dst row i = src row order[i].
__global__ void gather_rows_fp8_kernel(const uint8_t* __restrict__ src_q, const float* __restrict__ src_s,
                                       const int* __restrict__ order, int H, uint8_t* __restrict__ dst_q,
                                       float* __restrict__ dst_s) {
  const int i = blockIdx.x, tid = threadIdx.x;
  const int srow = order[i];
  const uint4 v = *reinterpret_cast<const uint4*>(src_q + static_cast<size_t>(srow) * H + tid * 16);
  *reinterpret_cast<uint4*>(dst_q + static_cast<size_t>(i) * H + tid * 16) = v;
  const int groups = H / 128;
  if (tid < groups) dst_s[static_cast<size_t>(i) * groups + tid] = src_s[static_cast<size_t>(srow) * groups + tid];
}

extern "C" int b200_gather_rows_fp8(const void* src_q, const float* src_scale, const int32_t* order,
                                    int num_rows, int hidden, void* dst_q, float* dst_scale, void* stream) {
  B200_REQUIRE(src_q && src_scale && order && dst_q && dst_scale, "gather_rows_fp8: null pointer");
  B200_REQUIRE(num_rows >= 0 && hidden > 0 && hidden % 512 == 0 && hidden <= 16384,
               "gather_rows_fp8: hidden %d must be a multiple of 512", hidden);
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(src_q) | reinterpret_cast<uintptr_t>(dst_q)) & 15) == 0,
               "gather_rows_fp8: buffers must be 16-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  if (num_rows == 0) return 0;
  gather_rows_fp8_kernel<<<num_rows, hidden / 16, 0, as_stream(stream)>>>(
      static_cast<const uint8_t*>(src_q), src_scale, order, hidden, static_cast<uint8_t*>(dst_q), dst_scale);
  B200_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int b200_moe_combine_add_rmsnorm(const void* y_sorted, const int32_t* row_of_pair,
                                            const float* topk_weights, void* x, const void* weight,
                                            float eps, int num_tokens, int hidden, int top_k, void* out,
                                            void* stream) {
  B200_REQUIRE(y_sorted && row_of_pair && topk_weights && x && weight && out,
               "moe_combine_add_rmsnorm: null pointer");
  B200_REQUIRE(num_tokens >= 0 && hidden > 0 && hidden % 256 == 0 && hidden <= 8192 && top_k > 0,
               "moe_combine_add_rmsnorm: bad dimensions T=%d H=%d K=%d", num_tokens, hidden, top_k);
  B200_REQUIRE(((reinterpret_cast<uintptr_t>(y_sorted) | reinterpret_cast<uintptr_t>(x) |
                 reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
               "moe_combine_add_rmsnorm: buffers must be 16-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  if (num_tokens == 0) return 0;
  B200_CUDA(launch_overlapped(moe_combine_add_rmsnorm_kernel, dim3(num_tokens), dim3(hidden / 8), 0, as_stream(stream),
                              static_cast<const __nv_bfloat16*>(y_sorted), row_of_pair, topk_weights, hidden, top_k,
                              static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(weight), eps,
                              static_cast<__nv_bfloat16*>(out)));
  return 0;
}

extern "C" int b200_act_quant_fp8(const void* x, const int32_t* row_of_pair, int num_tokens,
                                  int hidden, int top_k, void* xq, float* x_scale, void* stream) {
  B200_REQUIRE(x && xq && x_scale, "act_quant_fp8: null pointer");
  B200_REQUIRE(num_tokens >= 0 && hidden > 0 && hidden % 256 == 0 && hidden <= 8192,
               "act_quant_fp8: hidden %d must be a multiple of 256 and <= 8192", hidden);
  B200_REQUIRE(row_of_pair == nullptr || top_k > 0, "act_quant_fp8: top_k must be positive");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(xq) & 7) == 0,
               "act_quant_fp8: x must be 16-byte and xq 8-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  if (num_tokens == 0) return 0;
  act_quant_scatter_kernel<<<num_tokens, hidden / 8, 0, as_stream(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), row_of_pair, hidden, top_k, static_cast<uint8_t*>(xq),
      x_scale);
  B200_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int b200_moe_combine(const void* y_sorted, const int32_t* row_of_pair,
                                const float* topk_weights, int num_tokens, int hidden, int top_k,
                                void* out, void* stream) {
  B200_REQUIRE(y_sorted && row_of_pair && topk_weights && out, "moe_combine: null pointer");
  B200_REQUIRE(num_tokens >= 0 && hidden > 0 && hidden % 8 == 0 && hidden <= 8192 && top_k > 0,
               "moe_combine: bad dimensions T=%d H=%d K=%d", num_tokens, hidden, top_k);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(y_sorted) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
               "moe_combine: buffers must be 16-byte aligned");
  int rc = check_device(nullptr);
  if (rc) return rc;
  if (num_tokens == 0) return 0;
  moe_combine_kernel<<<num_tokens, hidden / 8, 0, as_stream(stream)>>>(
      static_cast<const __nv_bfloat16*>(y_sorted), row_of_pair, topk_weights, hidden, top_k,
      static_cast<__nv_bfloat16*>(out));
  B200_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int b200_moe_permute_gather_fp8(const int32_t* ids, int num_rows, int num_experts, int tile_experts,
                                           const void* src_q, const float* src_scale, int hidden,
                                           int32_t* sorted_ids, int32_t* row_of_id, int32_t* expert_offsets,
                                           void* tiles, int32_t* num_tiles, void* dst_q, float* dst_scale,
                                           void* workspace, size_t workspace_bytes, void* stream) {
  B200_REQUIRE(ids && src_q && src_scale && sorted_ids && row_of_id && expert_offsets && tiles && num_tiles &&
                   dst_q && dst_scale && workspace,
               "moe_permute_gather_fp8: null pointer");
  B200_REQUIRE(num_rows >= 0 && num_experts > 0 && num_experts <= 256 && tile_experts > 0 &&
                   tile_experts <= num_experts,
               "moe_permute_gather_fp8: rows %d, experts %d (at most 256), tile_experts %d", num_rows, num_experts,
               tile_experts);
  B200_REQUIRE(hidden > 0 && hidden % 128 == 0, "moe_permute_gather_fp8: hidden %d must be a multiple of 128", hidden);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(src_q) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst_q) & 15) == 0,
               "moe_permute_gather_fp8: row buffers must be 16-byte aligned");
  const size_t need = b200_moe_permute_workspace_bytes(num_rows, num_experts, 1);
  if (workspace_bytes < need) {
    set_detail("moe_permute_gather_fp8: workspace %zu < required %zu", workspace_bytes, need);
    return -kErrWorkspace;
  }
  int rc = check_device(nullptr);
  if (rc) return rc;
  cudaStream_t st = as_stream(stream);
  if (num_rows == 0) {
    // nothing received, but a GEMM that follows must not find the previous call's tiles
    B200_CUDA(cudaMemsetAsync(num_tiles, 0, sizeof(int32_t), st));
    B200_CUDA(cudaMemsetAsync(expert_offsets, 0, (static_cast<size_t>(num_experts) + 1) * sizeof(int32_t), st));
    return 0;
  }
  uint8_t* p = static_cast<uint8_t*>(workspace);
  int* err = reinterpret_cast<int*>(p);
  int* counts = reinterpret_cast<int*>(p + 256);
  int* rank = reinterpret_cast<int*>(p + 256 + ((static_cast<size_t>(num_experts) * 4 + 255) & ~size_t(255)));
  moe_rank_kernel<<<num_experts, kRankThreads, 0, st>>>(ids, num_rows, rank, counts);
  B200_CUDA(cudaGetLastError());
  const int threads = hidden / 16 < 256 ? (hidden / 16 < 32 ? 32 : hidden / 16) : 256;
  const size_t smem = (2 * static_cast<size_t>(num_experts) + 1) * sizeof(int);
  moe_scatter_rows_kernel<<<num_rows, threads, smem, st>>>(
      ids, rank, counts, num_experts, tile_experts, hidden, 128, sorted_ids, row_of_id, expert_offsets,
      static_cast<MoeTile*>(tiles), num_tiles, static_cast<const uint8_t*>(src_q), src_scale,
      static_cast<uint8_t*>(dst_q), dst_scale, err);
  B200_CUDA(cudaGetLastError());
  return 0;
}
