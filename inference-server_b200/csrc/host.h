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
