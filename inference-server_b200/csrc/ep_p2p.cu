// Expert-parallel exchange over peer memory: plumbing that lets the dispatch (scatter + quantise) and the
// return path (down-GEMM epilogue) write straight into the other GPUs' buffers over NVLink, instead of
// staging rows locally and calling a library all-to-all.  The reference is single-device and has no
// counterpart for anything in this file.
//
//   b200_ipc_export / b200_ipc_import / b200_ipc_close
//       share one device allocation ("arena") per rank between the processes of a node (CUDA IPC);
//   b200_ep_signal / b200_ep_wait / b200_ep_barrier
//       flag exchange that orders one rank's peer stores before another rank's reads.
//
// Protocol.  Every rank owns, per exchange phase, an array flags[world] in its arena and a local epoch
// counter.  signal: epoch += 1, then store the new epoch into flags[my_rank] of EVERY rank (system-scope
// release; the data stores were issued by earlier kernels of the same stream and are complete at that kernel
// boundary).  wait: spin, with an iteration limit, until every entry of the local flags is >= the local epoch
// (system-scope acquire).  All ranks run the same sequence of phases, so epochs agree; flags only grow, so a
// rank that runs ahead never blocks one that lags.  A wait that runs out records kErrDevPeerTimeout in the
// status word and returns: the step's results are then wrong and the host sees the code, but nothing hangs.
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "host.h"

namespace b200 {

constexpr uint32_t kEpWaitPolls = 1u << 20;  // x (>= 200 ns sleep + one system-scope load): of the order of a second

struct EpFlagPeers {
  int* flags[kMaxEpWorld];
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ int ep_bump_epoch(int* epoch) {
  __shared__ int e_sm;
  if (threadIdx.x == 0) {
    e_sm = *epoch + 1;
    *epoch = e_sm;
  }
  __syncthreads();
  return e_sm;
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Spins (bounded) until *flag reaches `want`.  The status block doubles as a small diagnostic: word 16 + r of
// a status array of at least 64 words accumulates the nanoseconds this rank spent waiting for rank r.
__device__ __forceinline__ void ep_wait_flag(const int* flag, int want, int* err, int peer) {
  bool ok = false;
  const unsigned long long t0 = global_ns();
  for (uint32_t i = 0; i < kEpWaitPolls; ++i) {
    if (ld_acquire_sys(flag) - want >= 0) {
      ok = true;
      break;
    }
    if (i > 64) __nanosleep(200);
  }
  if (!ok) set_error(err, kErrDevPeerTimeout);
  if (err != nullptr) atomicAdd(reinterpret_cast<unsigned int*>(err) + 16 + peer,
                                static_cast<unsigned int>((global_ns() - t0) & 0xffffffffu));
  __threadfence_system();
}

__global__ void ep_signal_kernel(const EpFlagPeers fp, int* epoch, int my_rank, int world) {
  const int e = ep_bump_epoch(epoch);
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(fp.flags[threadIdx.x] + my_rank, e);
  }
}

__global__ void ep_wait_kernel(const int* local_flags, const int* epoch, int world, int* err) {
  if (threadIdx.x < world) ep_wait_flag(local_flags + threadIdx.x, *epoch, err, threadIdx.x);
}

// signal + wait in one launch: thread r tells rank r, then waits for rank r.
__global__ void ep_barrier_kernel(const EpFlagPeers fp, const int* local_flags, int* epoch, int my_rank,
                                  int world, int* err) {
  const int e = ep_bump_epoch(epoch);
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(fp.flags[threadIdx.x] + my_rank, e);
    ep_wait_flag(local_flags + threadIdx.x, e, err, threadIdx.x);
  }
}

static int fill_flag_peers(void* const* flag_peers, int world, EpFlagPeers* fp, const char* who) {
  B200_REQUIRE(flag_peers && world >= 1 && world <= kMaxEpWorld, "%s: %d ranks (at most %d)", who, world, kMaxEpWorld);
  for (int r = 0; r < world; ++r) {
    B200_REQUIRE(flag_peers[r] && (reinterpret_cast<uintptr_t>(flag_peers[r]) & 3) == 0,
                 "%s: flag array of rank %d null or unaligned", who, r);
    fp->flags[r] = static_cast<int*>(flag_peers[r]);
  }
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_ep_signal(void* const* flag_peers, int32_t* epoch, int ep_rank, int ep_world, void* stream) {
  EpFlagPeers fp{};
  int rc = fill_flag_peers(flag_peers, ep_world, &fp, "ep_signal");
  if (rc) return rc;
  B200_REQUIRE(epoch && ep_rank >= 0 && ep_rank < ep_world, "ep_signal: null epoch or rank %d of %d", ep_rank, ep_world);
  ep_signal_kernel<<<1, 32, 0, as_stream(stream)>>>(fp, epoch, ep_rank, ep_world);
  B200_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int b200_ep_wait(const int32_t* local_flags, const int32_t* epoch, int ep_world, void* status_word,
                            void* stream) {
  B200_REQUIRE(local_flags && epoch && ep_world >= 1 && ep_world <= kMaxEpWorld, "ep_wait: null pointer or %d ranks",
               ep_world);
  ep_wait_kernel<<<1, 32, 0, as_stream(stream)>>>(local_flags, epoch, ep_world, static_cast<int*>(status_word));
  B200_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int b200_ep_barrier(void* const* flag_peers, int32_t* epoch, int ep_rank, int ep_world,
                               void* status_word, void* stream) {
  EpFlagPeers fp{};
  int rc = fill_flag_peers(flag_peers, ep_world, &fp, "ep_barrier");
  if (rc) return rc;
  B200_REQUIRE(epoch && ep_rank >= 0 && ep_rank < ep_world, "ep_barrier: null epoch or rank %d of %d", ep_rank, ep_world);
  ep_barrier_kernel<<<1, 32, 0, as_stream(stream)>>>(fp, fp.flags[ep_rank], epoch, ep_rank, ep_world,
                                                     static_cast<int*>(status_word));
  B200_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------ CUDA IPC --
extern "C" int b200_ipc_export(const void* ptr, void* handle_out, uint64_t* offset_out) {
  B200_REQUIRE(ptr && handle_out && offset_out, "ipc_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the ABI");
  typedef CUresult (*GetRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  B200_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres));
  B200_REQUIRE(fn != nullptr && qres == cudaDriverEntryPointSuccess, "ipc_export: cuMemGetAddressRange unavailable");
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult cr = reinterpret_cast<GetRangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  B200_REQUIRE(cr == CUDA_SUCCESS, "ipc_export: cuMemGetAddressRange failed (%d)", static_cast<int>(cr));
  cudaIpcMemHandle_t h;
  B200_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(handle_out, &h, sizeof(h));
  *offset_out = reinterpret_cast<CUdeviceptr>(ptr) - base;
  return 0;
}

extern "C" int b200_ipc_import(const void* handle, uint64_t offset, void** base_out, void** ptr_out) {
  B200_REQUIRE(handle && base_out && ptr_out, "ipc_import: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* base = nullptr;
  B200_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *base_out = base;
  *ptr_out = static_cast<uint8_t*>(base) + offset;
  return 0;
}

extern "C" int b200_ipc_close(void* base) {
  B200_REQUIRE(base, "ipc_close: null pointer");
  B200_CUDA(cudaIpcCloseMemHandle(base));
  return 0;
}
