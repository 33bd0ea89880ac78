// Host-side support for the C-ABI: device check, TMA tensor-map cache, error
// text.  Nothing here launches a kernel or allocates device memory.

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "common.cuh"
#include "host.h"

namespace b200 {

static thread_local char g_detail[512] = "";

void set_detail(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_detail, sizeof(g_detail), fmt, ap);
  va_end(ap);
}
const char* get_detail() { return g_detail; }

int cuda_fail(cudaError_t e, const char* where) {
  set_detail("%s: %s", where, cudaGetErrorString(e));
  return -kErrCuda;
}

// Per-device facts and per-(kernel, device) attribute calls, remembered under one mutex so that concurrent
// first calls from several host threads neither race nor repeat the driver call.
struct DeviceFacts {
  int device, major, sm_count;
};
static std::mutex g_dev_mu;
static std::vector<DeviceFacts> g_devices;
struct KernelAttr {
  const void* kernel;
  int device, bytes;
};
static std::vector<KernelAttr> g_kernel_attrs;

static int device_facts(DeviceFacts* out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  std::lock_guard<std::mutex> lock(g_dev_mu);
  for (const DeviceFacts& f : g_devices)
    if (f.device == dev) {
      *out = f;
      return 0;
    }
  DeviceFacts f{dev, 0, 0};
  e = cudaDeviceGetAttribute(&f.major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(major)");
  e = cudaDeviceGetAttribute(&f.sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute(sm count)");
  g_devices.push_back(f);
  *out = f;
  return 0;
}

int check_device(int* device_out) {
  DeviceFacts f;
  int rc = device_facts(&f);
  if (rc) return rc;
  if (f.major != 10) {
    set_detail("device %d has compute capability %d.x; this library is built for sm_100a only", f.device,
               f.major);
    return -kErrUnsupported;
  }
  if (device_out) *device_out = f.device;
  return 0;
}

bool overlapped_launch_enabled() {
  static const bool enabled = [] {
    const char* v = getenv("B200_SERIAL_LAUNCH");
    return !(v && v[0] != '\0' && v[0] != '0');
  }();
  return enabled;
}

int device_sm_count(int* out) {
  DeviceFacts f;
  int rc = device_facts(&f);
  if (rc) return rc;
  *out = f.sm_count > 0 ? f.sm_count : 148;
  return 0;
}

int ensure_dynamic_smem(const void* kernel, int bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  std::lock_guard<std::mutex> lock(g_dev_mu);
  for (const KernelAttr& a : g_kernel_attrs)
    if (a.kernel == kernel && a.device == dev && a.bytes >= bytes) return 0;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(max dynamic shared memory)");
  g_kernel_attrs.push_back(KernelAttr{kernel, dev, bytes});
  return 0;
}

// ------------------------------------------------------- tensor-map cache --
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct MapKey {
  int device;
  const void* base;
  uint64_t rows, cols;
  int elem_bytes;
  uint32_t box_rows, box_cols;
  bool operator==(const MapKey& o) const {
    return device == o.device && base == o.base && rows == o.rows && cols == o.cols &&
           elem_bytes == o.elem_bytes && box_rows == o.box_rows && box_cols == o.box_cols;
  }
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
};

static std::mutex g_map_mu;
static std::vector<MapEntry> g_maps;
static EncodeTiledFn g_encode = nullptr;

int get_tensor_map_2d(const void* base, uint64_t rows, uint64_t cols, int elem_bytes,
                      uint32_t box_rows, uint32_t box_cols, CUtensorMap* out) {
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaGetDevice");
  MapKey key{dev, base, rows, cols, elem_bytes, box_rows, box_cols};
  std::lock_guard<std::mutex> lock(g_map_mu);
  for (const MapEntry& e : g_maps) {
    if (e.key == key) {
      *out = e.map;
      return 0;
    }
  }
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    ce = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (ce != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
      set_detail("cuTensorMapEncodeTiled is not available from the driver");
      return -kErrTensorMap;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  if (box_cols * static_cast<uint32_t>(elem_bytes) != 128u || box_rows == 0 || box_rows > 256 ||
      (reinterpret_cast<uintptr_t>(base) & 15) != 0 || (cols * elem_bytes) % 16 != 0) {
    set_detail("tensor map: base %p rows %llu cols %llu elem %d box %ux%u is not encodable", base,
               (unsigned long long)rows, (unsigned long long)cols, elem_bytes, box_rows, box_cols);
    return -kErrTensorMap;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {cols * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  MapEntry entry;
  entry.key = key;
  CUresult r = g_encode(&entry.map,
                        elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8,
                        2, const_cast<void*>(base), gdim, gstride, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_detail("cuTensorMapEncodeTiled failed with CUresult %d (base %p rows %llu cols %llu)", (int)r,
               base, (unsigned long long)rows, (unsigned long long)cols);
    return -kErrTensorMap;
  }
  if (g_maps.size() >= 4096) g_maps.erase(g_maps.begin(), g_maps.begin() + 2048);
  g_maps.push_back(entry);
  *out = entry.map;
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_abi_version(void) { return 1; }

extern "C" const char* b200_strerror(int code) {
  switch (code < 0 ? -code : code) {
    case kErrOk: return "ok";
    case kErrBadArg: return "bad argument (null pointer, shape or alignment)";
    case kErrUnsupported: return "unsupported device or configuration (sm_100a required)";
    case kErrWorkspace: return "workspace too small";
    case kErrCuda: return "CUDA runtime error";
    case kErrTensorMap: return "TMA tensor map could not be encoded";
    case kErrDevBadBlockId: return "device: block table entry outside the pool";
    case kErrDevBadCtxLen: return "device: context length or position outside the block table";
    case kErrDevWaitTimeout: return "device: a bounded barrier wait ran out";
    case kErrDevBadExpert: return "device: expert id outside [0, num_experts)";
    case kErrDevPeerTimeout: return "device: a bounded wait for another rank's flag ran out";
    default: return "unknown error";
  }
}

extern "C" const char* b200_last_error_detail(void) { return get_detail(); }

// Copies the device status word back and returns it negated (0 = clean).
// This is the one entry point that synchronises the stream.
extern "C" int b200_read_status(const void* status_word, void* stream) {
  if (status_word == nullptr) {
    set_detail("read_status: null pointer");
    return -kErrBadArg;
  }
  int v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, status_word, sizeof(int), cudaMemcpyDeviceToHost, as_stream(stream));
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(status)");
  e = cudaStreamSynchronize(as_stream(stream));
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
  return -v;
}
