// Host-side helpers shared by the C-ABI translation units: argument checks,
// device capability check, and a mutex-guarded cache of TMA tensor maps.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "b200_decode.h"

namespace b200 {

// Returns 0 when the current device is sm_100-class, else a negative error.
int check_device(int* device_out);

// Raises a kernel's dynamic shared-memory limit to `bytes` once per (kernel, device); later calls for the same
// pair only look the pair up.  Safe to call from several host threads.  Returns 0 or a negative error code.
int ensure_dynamic_smem(const void* kernel, int bytes);

// Multiprocessor count of the current device (cached per device, thread-safe).
int device_sm_count(int* out);

// Looks up (or encodes and caches) a 2-D row-major tensor map:
//   rows x cols elements of `elem_bytes` (1 = uint8, 2 = bf16), row pitch =
//   cols * elem_bytes, box = box_rows x box_cols, 128-byte swizzle.
// box_cols * elem_bytes must be 128.  Returns 0 or a negative error code.
int get_tensor_map_2d(const void* base, uint64_t rows, uint64_t cols, int elem_bytes,
                      uint32_t box_rows, uint32_t box_cols, CUtensorMap* out);

// Records the last CUDA error text for b200_last_error_detail().
int cuda_fail(cudaError_t e, const char* where);
void set_detail(const char* fmt, ...);
const char* get_detail();

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// True unless the environment variable B200_SERIAL_LAUNCH is set to a non-zero value (read once).
bool overlapped_launch_enabled();

// Launches a kernel that begins with grid_dep_wait() (common.cuh) as a programmatic dependent of the kernel before
// it in the stream: its blocks may be placed on the multiprocessors while that kernel drains and they hold at
// grid_dep_wait() until it has completed and its writes are visible, which takes the launch latency and the
// block placement off the critical path between two kernels.  Captured into a CUDA graph the edge becomes a
// programmatic dependency.  Only for kernels whose every thread executes grid_dep_wait() before it touches
// global memory or returns.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                     Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlapped_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace b200

#define B200_REQUIRE(cond, ...)            \
  do {                                     \
    if (!(cond)) {                         \
      ::b200::set_detail(__VA_ARGS__);     \
      return -::b200::kErrBadArg;          \
    }                                      \
  } while (0)

#define B200_CUDA(expr)                                              \
  do {                                                               \
    cudaError_t e__ = (expr);                                        \
    if (e__ != cudaSuccess) return ::b200::cuda_fail(e__, #expr);    \
  } while (0)
