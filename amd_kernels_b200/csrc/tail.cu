// The layer's fused tail: slot sum (+ shared expert) -> residual add -> Gemma RMSNorm -> MXFP8 quantisation of the next
// layer's input, one pass over the slots instead of a reduce kernel followed by a norm kernel (the single-GPU form of
// the reference's slots4_reduce_scatter_add_rmsnorm_mxfp8, amd_kernels/collectives/pull_collectives_ranks4/README.md:25-27;
// contract: .../pull_collectives_ranks4/reference.py:74-91 slots4_reduce_scatter_reference for the sum and
// amd_kernels/norm/gemma_add_rmsnorm_h6144/reference.py steps 2-4 for the rest).
//
// Per token row of 6144 columns:
//   x   = bf16( (((s0 + s1) + s2) + s3) (+ shared) )      fp32 adds in slot order, one rounding
//   s   = fp32(x) + fp32(residual);  residual_out = bf16(s)
//   y   = (s * rstd) * (weight + 1),  rstd = 1 / sqrt(sum(s^2) / 6144 + eps)     (the norm reads the fp32 s)
//   out = bf16(y)                                                                 (optional)
//   per 32 columns of y: a = max(max|y|, 2^-126), scale byte = clamp(ceil(log2(a / 448)) + 127, 0, 254),
//   code = e4m3(y * 2^(127 - byte)), round to nearest even, saturating                            (optional)
// One 256-thread CTA per row, 24 columns per thread as three 16-byte vectors; the sum of squares is reduced in a fixed
// order (thread-local, warp tree, then the eight warp sums in warp order), so results repeat bit for bit.
#include "common.cuh"

namespace b200moe {

__device__ __forceinline__ void unpack_bf16x8(const uint4 v, float (&f)[8]) {
  const uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __uint_as_float(r[j] << 16);
    f[2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    o[j] = *reinterpret_cast<const uint32_t*>(&p);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// clamp(ceil(log2(a / 448)) + 127, 0, 254) for a >= 2^-126 (a may be +inf): the division rounded to fp32, then the
// exact ceiling of its base-2 logarithm read from the bits (subnormal quotients included).
__device__ __forceinline__ int tail_mxfp8_scale(float a) {
  const uint32_t u = __float_as_uint(__fdiv_rn(a, 448.0f));
  const int ef = static_cast<int>((u >> 23) & 255u);
  const uint32_t m = u & 0x7fffffu;
  int sb = ef ? ef + (m != 0u) : (m > 0x400000u ? 1 : 0);
  return sb > 254 ? 254 : sb;
}

__global__ void __launch_bounds__(256) tail_kernel(const uint4* __restrict__ slots, const uint4* __restrict__ shared,
                                                   const uint4* __restrict__ residual, const uint4* __restrict__ weight,
                                                   float eps, uint4* __restrict__ residual_out, uint4* __restrict__ out,
                                                   uint2* __restrict__ codes8, uint8_t* __restrict__ scales8) {
  pdl_enter(slots, shared, residual);
  constexpr int kVecPerRow = kH / 8, kIters = kH / 8 / 256;  // 768 vectors per row, 3 per thread
  __shared__ float warp_sum[8];
  const int64_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float s[kIters][8];
  float ss = 0.0f;
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int c = it * 256 + threadIdx.x;
    float acc[8], v[8];
    unpack_bf16x8(__ldcg(slots + (t * kTopK) * kVecPerRow + c), acc);
#pragma unroll
    for (int k = 1; k < kTopK; ++k) {
      unpack_bf16x8(__ldcg(slots + (t * kTopK + k) * kVecPerRow + c), v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = acc[j] + v[j];
    }
    if (shared != nullptr) {
      unpack_bf16x8(__ldcg(shared + t * kVecPerRow + c), v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = acc[j] + v[j];
    }
    unpack_bf16x8(__ldcg(residual + t * kVecPerRow + c), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float x = __bfloat162float(__float2bfloat16_rn(acc[j]));  // the combine rounds once, the norm reads bf16 x
      s[it][j] = x + v[j];
      ss = fmaf(s[it][j], s[it][j], ss);
    }
    residual_out[t * kVecPerRow + c] = pack_bf16x8(s[it]);
  }
#pragma unroll
  for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if (lane == 0) warp_sum[warp] = ss;
  __syncthreads();
  float total = 0.0f;
#pragma unroll
  for (int w = 0; w < 8; ++w) total += warp_sum[w];
  const float rstd = __frcp_rn(__fsqrt_rn(__fdiv_rn(total, static_cast<float>(kH)) + eps));
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int c = it * 256 + threadIdx.x;
    float wv[8], y[8];
    unpack_bf16x8(__ldg(weight + c), wv);
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      y[j] = (s[it][j] * rstd) * (wv[j] + 1.0f);
      amax = fmaxf(amax, fabsf(y[j]));  // fmaxf skips a NaN operand
    }
    if (out != nullptr) out[t * kVecPerRow + c] = pack_bf16x8(y);
    if (codes8 != nullptr) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const int sb = tail_mxfp8_scale(fmaxf(amax, 1.17549435e-38f));
      const float inv = e8m0_value(static_cast<uint32_t>(254 - sb));  // 2^(127 - sb)
      const uint32_t w0 = cvt_e4m3x2(y[0] * inv, y[1] * inv) | (cvt_e4m3x2(y[2] * inv, y[3] * inv) << 16);
      const uint32_t w1 = cvt_e4m3x2(y[4] * inv, y[5] * inv) | (cvt_e4m3x2(y[6] * inv, y[7] * inv) << 16);
      codes8[t * kVecPerRow + c] = make_uint2(w0, w1);
      if ((lane & 3) == 0) scales8[t * (kH / 32) + (c >> 2)] = static_cast<uint8_t>(sb);
    }
  }
}

}  // namespace b200moe

extern "C" int b200moe_reduce_slots_add_rmsnorm_quant(const void* slots_bf16, const void* shared_bf16,
                                                      const void* residual_bf16, const void* weight_bf16, float eps,
                                                      int64_t tokens, void* residual_out_bf16, void* out_bf16,
                                                      uint8_t* codes8, uint8_t* scales8, void* stream) {
  using namespace b200moe;
  if (!slots_bf16 || !residual_bf16 || !weight_bf16 || !residual_out_bf16 || tokens < 0) return B200MOE_E_ARG;
  if ((codes8 != nullptr) != (scales8 != nullptr)) return B200MOE_E_ARG;
  const void* aligned[] = {slots_bf16, shared_bf16, residual_bf16, weight_bf16, residual_out_bf16, out_bf16, codes8};
  for (const void* p : aligned)
    if (reinterpret_cast<uintptr_t>(p) & 15) return B200MOE_E_ALIGN;
  if (tokens == 0) return 0;
  B200MOE_LAUNCH(tail_kernel, static_cast<unsigned>(tokens), 256, 0, static_cast<cudaStream_t>(stream),
                 static_cast<const uint4*>(slots_bf16), static_cast<const uint4*>(shared_bf16),
                 static_cast<const uint4*>(residual_bf16), static_cast<const uint4*>(weight_bf16), eps,
                 static_cast<uint4*>(residual_out_bf16), static_cast<uint4*>(out_bf16), reinterpret_cast<uint2*>(codes8),
                 scales8);
  return 0;
}
