// Slot reduce: out = bf16(((0 + s0) + s1) + s2) + s3 (+ shared)) in fp32, one rounding, 8 columns per thread.
#include "common.cuh"

namespace b200moe {

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4 v) {
  const uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    acc[2 * j] = acc[2 * j] + __uint_as_float(r[j] << 16);
    acc[2 * j + 1] = acc[2 * j + 1] + __uint_as_float(r[j] & 0xffff0000u);
  }
}

// `index` (optional): row of `slots` that holds pair 4*token+slot, for slot rows that sit in another order (rows that came
// back from other ranks in send order); without it pair q is row q.
__global__ void __launch_bounds__(256) reduce_slots_kernel(const uint4* __restrict__ slots,
                                                           const int32_t* __restrict__ index,
                                                           const uint4* __restrict__ shared, int64_t n_vec,
                                                           uint4* __restrict__ out) {
  pdl_enter(slots, index, shared);
  constexpr int kVecPerRow = kH / 8;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const int64_t t = i / kVecPerRow, c = i % kVecPerRow;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll
  for (int s = 0; s < kTopK; ++s) {
    const int64_t row = index ? static_cast<int64_t>(__ldcg(index + t * kTopK + s)) : t * kTopK + s;
    add_bf16x8(acc, __ldcg(slots + row * kVecPerRow + c));
  }
  if (shared) add_bf16x8(acc, __ldcg(shared + i));
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    o[j] = *reinterpret_cast<const uint32_t*>(&p);
  }
  out[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace b200moe

extern "C" int b200moe_reduce_slots(const void* slots_bf16, const void* shared_bf16, int64_t tokens, void* out_bf16,
                                    void* stream) {
  using namespace b200moe;
  if (!slots_bf16 || !out_bf16 || tokens < 0) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(slots_bf16) & 15) || (reinterpret_cast<uintptr_t>(out_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(shared_bf16) & 15))
    return B200MOE_E_ALIGN;
  if (tokens == 0) return 0;
  const int64_t n_vec = tokens * (kH / 8);
  B200MOE_LAUNCH(reduce_slots_kernel, static_cast<unsigned>((n_vec + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream), static_cast<const uint4*>(slots_bf16), static_cast<const int32_t*>(nullptr), static_cast<const uint4*>(shared_bf16), n_vec, static_cast<uint4*>(out_bf16));
  return 0;
}

extern "C" int b200moe_reduce_rows(const void* rows_bf16, const int32_t* index, const void* shared_bf16, int64_t tokens,
                                   void* out_bf16, void* stream) {
  using namespace b200moe;
  if (!rows_bf16 || !index || !out_bf16 || tokens < 0) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(rows_bf16) & 15) || (reinterpret_cast<uintptr_t>(out_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(shared_bf16) & 15))
    return B200MOE_E_ALIGN;
  if (tokens == 0) return 0;
  const int64_t n_vec = tokens * (kH / 8);
  B200MOE_LAUNCH(reduce_slots_kernel, static_cast<unsigned>((n_vec + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream),
                 static_cast<const uint4*>(rows_bf16), index, static_cast<const uint4*>(shared_bf16), n_vec,
                 static_cast<uint4*>(out_bf16));
  return 0;
}
