// Shared constants and device helpers of libb200moe (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200_moe.h"

namespace b200moe {

constexpr int kH = B200MOE_H;        // hidden size
constexpr int kI = B200MOE_I;        // intermediate size (per expert, after SwiGLU)
constexpr int kTopK = B200MOE_TOPK;
constexpr int kMaxE = B200MOE_E;

constexpr int kW13Tiles = 2 * kI / 128;  // 12 tiles of 64 gate + 64 up rows per expert
constexpr int kW2Tiles = kH / 128;       // 48
constexpr int kK1Tiles = kH / 256;       // 24 K-tiles (256 elements = 128 bytes) in GEMM1
constexpr int kK2Tiles = kI / 256;       // 3 in GEMM2
constexpr int kAtomBytes = 512;          // one scale atom
constexpr int kTileRecordBytes = 128 * 128 + 2 * kAtomBytes;  // one weight tile (swizzled codes + scales) in HBM

#define B200MOE_CHECK_LAUNCH()                        \
  do {                                                \
    cudaError_t e__ = cudaGetLastError();             \
    if (e__ != cudaSuccess) return static_cast<int>(e__); \
  } while (0)

// Programmatic dependent launch: every kernel of the library is launched with the programmatic-serialization attribute,
// lets its successor start early (launch_dependents) and waits for its predecessors' memory (wait) before it touches
// global memory. A successor therefore overlaps its launch latency and set-up with the tail of the kernel before it.
//
// Two rules follow from a kernel being resident BEFORE its inputs exist: (1) pointers to data a predecessor writes are
// laundered through an empty asm after the wait, so the compiler cannot hoist a load (const __restrict__ loads count as
// invariant and would otherwise move above the wait); (2) such data is read with L2-coherent loads (ld.global.cg, TMA or
// bulk copies), never through the non-coherent L1 path, which may hold lines an older kernel fetched on the same SM.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename T>
__device__ __forceinline__ void launder(T& p) {  // T is a (possibly __restrict__) pointer type
  asm volatile("" : "+l"(p)::"memory");
}
// launch the successor early, wait for the predecessors, then forget everything known about the given pointers
template <typename... P>
__device__ __forceinline__ void pdl_enter(P&... ptrs) {
  pdl_launch_dependents();
  pdl_wait();
  (launder(ptrs), ...);
}

// ask L2 to fetch `bytes` (a multiple of 16) at a 16-byte aligned global address; no register or shared-memory destination
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(p)), "r"(bytes) : "memory");
}

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// kernels outside the per-call chain (load-time preshuffle, cross-check kernels) use ordinary stream order
#define B200MOE_LAUNCH_PLAIN(kernel, grid, block, smem, stream, ...)          \
  do {                                                                        \
    kernel<<<grid, block, smem, stream>>>(__VA_ARGS__);                       \
    B200MOE_CHECK_LAUNCH();                                                   \
  } while (0)

#define B200MOE_LAUNCH(kernel, grid, block, smem, stream, ...)                                        \
  do {                                                                                                \
    cudaError_t e__ = b200moe::launch_pdl(kernel, grid, block, smem, stream, __VA_ARGS__);            \
    if (e__ != cudaSuccess) return static_cast<int>(e__);                                             \
  } while (0)

__device__ __forceinline__ float e2m1_value(uint32_t code) {
  // {0,.5,1,1.5,2,3,4,6} with the sign in bit 3
  const uint32_t m = code & 7u;
  float v = (m < 2u) ? 0.5f * static_cast<float>(m)
                     : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
  return (code & 8u) ? -v : v;
}

__device__ __forceinline__ float e8m0_value(uint32_t byte) {
  // 2^(byte-127); byte 0 is 2^-127 (a subnormal float)
  return byte ? __uint_as_float(byte << 23) : __uint_as_float(0x00400000u);
}

// "Quark even" block scale from the block's absolute maximum: max(1, (bits(amax) - 0x00E00000) >> 23), arithmetic shift.
__device__ __forceinline__ int quark_even_e8m0(float amax) {
  int e = (static_cast<int>(__float_as_uint(amax)) - 0x00E00000) >> 23;
  return e < 1 ? 1 : e;
}

// E2M1 code of v at scale byte e: number of midpoints below |v| / 2^(e-127), ties to the even code, sign from the bit.
__device__ __forceinline__ uint32_t e2m1_code(float v, int e) {
  const float inv = __uint_as_float(static_cast<uint32_t>(254 - e) << 23);  // 2^(127-e), e <= 253
  const float a = fabsf(v) * inv;
  uint32_t c = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f);
  return c | ((__float_as_uint(v) >> 31) << 3);
}

// ceil_pow2(amax / 448) as an E8M0 byte, at least 1 (the reference's shared_mxfp8_quant_ref)
__device__ __forceinline__ int mxfp8_scale(float amax) {
  const uint32_t u = __float_as_uint(__fdiv_rn(amax, 448.0f));
  int e = static_cast<int>((u >> 23) & 255u);
  if ((u & 0x7fffffu) != 0u && e < 255) ++e;
  return e < 1 ? 1 : e;
}

// two E4M3 codes: `lo` in the low byte, `hi` in the high byte; round to nearest even, saturating
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t out;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(out) : "f"(hi), "f"(lo));
  return out;
}

// two E2M1 codes in one byte: `lo` in the low nibble, `hi` in the high nibble; round to nearest even, saturating.
// Same codes as e2m1_code on a value already divided by the block scale (ties go to the even code, -0 keeps its sign).
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
  uint16_t out;
  asm("{\n.reg .b8 t;\ncvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\ncvt.u16.u8 %0, t;\n}\n" : "=h"(out) : "f"(hi), "f"(lo));
  return out;
}

__device__ __forceinline__ float swiglu_oai(float g, float u) {
  g = fminf(g, 7.0f);
  u = fminf(fmaxf(u, -7.0f), 7.0f);
  const float sig = __fdividef(1.0f, 1.0f + __expf(-1.702f * g));  // exp2 + rcp approximations, as the reference kernels
  return g * sig * (u + 1.0f);
}

// byte offset of scale j (0..3) of row r (0..127) inside a 512-byte scale atom
__device__ __host__ __forceinline__ int atom_offset(int r, int j) { return (r & 31) * 16 + (r >> 5) * 4 + j; }

// 256 threads (t = 0..255, whole warps) quantise one bf16 row of kH values to MXFP4: 3072 code bytes to `dst` and the 192
// scale bytes into the row's cells of its block's scale atoms (`sdst` = atom 0 + atom_offset(row in block, 0)). The three
// 16-byte loads of a thread are in flight together. `src` null: a padding row (zero codes, the scale byte of a zero block).
__device__ __forceinline__ void quant_row_to_atoms(const uint4* src, uint32_t* dst, uint8_t* sdst, int t) {
  constexpr int kIters = kH / 8 / 256;  // 3
  const int lane = t & 31;
  if (src == nullptr) {
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      const int idx = it * 256 + t;
      dst[idx] = 0u;
      if ((lane & 15) == 0) *reinterpret_cast<uint32_t*>(sdst + (idx >> 4) * kAtomBytes) = 0x01010101u;
    }
    return;
  }
  uint4 raw[kIters];
#pragma unroll
  for (int it = 0; it < kIters; ++it) raw[it] = __ldcg(src + it * 256 + t);
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int idx = it * 256 + t;
    const uint32_t rr[4] = {raw[it].x, raw[it].y, raw[it].z, raw[it].w};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = __uint_as_float(rr[j] << 16);
      v[2 * j + 1] = __uint_as_float(rr[j] & 0xffff0000u);
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const int e = quark_even_e8m0(amax);
    const float inv = __uint_as_float(static_cast<uint32_t>(254 - e) << 23);  // 2^(127-e), exact
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) packed |= cvt_e2m1x2(v[2 * j] * inv, v[2 * j + 1] * inv) << (8 * j);
    dst[idx] = packed;
    // 4 lanes share a 32-element block, 16 lanes one scale atom's 4 bytes: lanes 0 and 16 gather their neighbours' bytes
    uint32_t sc = static_cast<uint32_t>(e);
    sc |= __shfl_down_sync(0xffffffffu, sc, 4) << 8;
    sc |= __shfl_down_sync(0xffffffffu, sc, 8) << 16;
    if ((lane & 15) == 0) *reinterpret_cast<uint32_t*>(sdst + (idx >> 4) * kAtomBytes) = sc;
  }
}

// The same for a row that is already quantised (row-major codes / scales of its token): copy and re-lay the scales.
__device__ __forceinline__ void copy_row_to_atoms(const uint8_t* codes, const uint8_t* scales, uint32_t* dst, uint8_t* sdst,
                                                  int t) {
  constexpr int kIters = kH / 8 / 256;  // 3 x 4 bytes of codes per thread
#pragma unroll
  for (int it = 0; it < kIters; ++it) dst[it * 256 + t] = __ldcg(reinterpret_cast<const uint32_t*>(codes) + it * 256 + t);
  if (t < kH / 128) *reinterpret_cast<uint32_t*>(sdst + t * kAtomBytes) = __ldcg(reinterpret_cast<const uint32_t*>(scales) + t);
}

}  // namespace b200moe
