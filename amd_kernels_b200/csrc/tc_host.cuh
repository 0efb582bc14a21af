// Host-side helpers of the tensor-core kernels: tensor-map encoding through the driver entry point, SM count.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/b200_moe.h"

namespace b200moe {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// byte matrix [rows][row_bytes], boxes of 128 bytes x box_rows, 128B swizzle
static inline int make_map(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return B200MOE_E_DRIVER;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : B200MOE_E_DRIVER;
}

constexpr int kMaxDevices = 64;

// SM count of the CURRENT device, looked up once per device (a process may drive several GPUs through this library).
static inline int sm_count() {
  static std::mutex mu;
  static int counts[kMaxDevices] = {};
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (counts[dev] == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    counts[dev] = v;
  }
  return counts[dev];
}

// Function attributes (dynamic shared-memory size, carve-out) belong to a device: `configure` runs once per device and
// kernel instantiation, with that device current, under a lock. One instance per launch-site template instantiation.
struct PerDeviceOnce {
  std::mutex mu;
  bool done[kMaxDevices] = {};
  template <typename F>
  int run(F&& configure) {
    int dev = 0;
    const cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= kMaxDevices) return B200MOE_E_ARG;
    std::lock_guard<std::mutex> lock(mu);
    if (done[dev]) return 0;
    const int r = configure();
    if (r == 0) done[dev] = true;
    return r;
  }
};


static inline bool misaligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; }

}  // namespace b200moe
