// CUDA-core versions of the two grouped GEMMs, reading checkpoint-layout weights and row-major activations.
// They produce the same outputs in the same layouts as the tcgen05 kernels and serve as an on-GPU cross-check of those
// kernels and of the weight preshuffle at sizes the CPU oracle cannot reach. The product path never selects them.
#include "common.cuh"

namespace b200moe {

// sum over 32 elements of code products, scaled by both block scales
__device__ __forceinline__ float dot32(const uint4 wq, const float* __restrict__ xv, float wscale) {
  const uint32_t r[4] = {wq.x, wq.y, wq.z, wq.w};
  float acc = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int n = 0; n < 8; ++n) acc = fmaf(e2m1_value((r[j] >> (4 * n)) & 15u), xv[8 * j + n], acc);
  return acc * wscale;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// grid (rows, 768/32); 256 threads: warp w computes intermediate columns i0 + 4w .. i0 + 4w + 3 of one sorted row
__global__ void __launch_bounds__(256) gemm1_simt_kernel(const uint8_t* __restrict__ w13, const uint8_t* __restrict__ s13,
                                                         const uint8_t* __restrict__ codes,
                                                         const uint8_t* __restrict__ scales,
                                                         const int32_t* __restrict__ sorted_ids,
                                                         const int32_t* __restrict__ block_expert,
                                                         const int32_t* __restrict__ num_valid,
                                                         const int32_t* __restrict__ rows, int bm, int64_t tokens,
                                                         uint8_t* __restrict__ hq, uint8_t* __restrict__ sfh) {
  __shared__ float xs[kH];
  __shared__ float hval[32];
  const int64_t row = rows ? rows[blockIdx.x] : blockIdx.x;
  if (row >= num_valid[0]) return;
  const int64_t token = sorted_ids[row] & 0x00ffffff;
  const bool pad = token >= tokens;
  const int e = block_expert[row / bm];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int k = threadIdx.x; k < kH; k += 256) {
    float v = 0.0f;
    if (!pad) {
      const uint32_t byte = codes[token * (kH / 2) + (k >> 1)];
      v = e2m1_value((byte >> ((k & 1) * 4)) & 15u) * e8m0_value(scales[token * (kH / 32) + (k >> 5)]);
    }
    xs[k] = v;
  }
  __syncthreads();
  const int i0 = blockIdx.y * 32;
#pragma unroll 1
  for (int j = 0; j < 4; ++j) {
    const int i = i0 + warp * 4 + j;
    float acc[2] = {0.0f, 0.0f};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int64_t wrow = static_cast<int64_t>(e) * 2 * kI + half * kI + i;
      const uint4* wq = reinterpret_cast<const uint4*>(w13 + wrow * (kH / 2));
      const uint8_t* ws = s13 + wrow * (kH / 32);
      for (int blk = lane; blk < kH / 32; blk += 32) acc[half] += dot32(wq[blk], xs + blk * 32, e8m0_value(ws[blk]));
      acc[half] = warp_sum(acc[half]);
    }
    if (lane == 0) hval[warp * 4 + j] = swiglu_oai(acc[0], acc[1]);
  }
  __syncthreads();
  if (warp == 0) {
    const float h = hval[lane];
    float amax = fabsf(h);
#pragma unroll
    for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const int sc = quark_even_e8m0(amax);
    uint32_t code = e2m1_code(h, sc);
    code |= __shfl_down_sync(0xffffffffu, code, 1) << 4;
    if ((lane & 1) == 0) hq[row * (kI / 2) + (i0 >> 1) + (lane >> 1)] = static_cast<uint8_t>(code);
    if (lane == 0) {
      const int g = blockIdx.y;  // 32-column group 0..23
      sfh[((row / bm) * (kI / 128) + (g >> 2)) * kAtomBytes + atom_offset(static_cast<int>(row % bm), g & 3)] =
          static_cast<uint8_t>(sc);
    }
  }
}

// grid (rows, 6144/64); 256 threads: warp w computes output columns n0 + 8w .. n0 + 8w + 7
__global__ void __launch_bounds__(256) gemm2_simt_kernel(const uint8_t* __restrict__ w2, const uint8_t* __restrict__ s2,
                                                         const uint8_t* __restrict__ hq, const uint8_t* __restrict__ sfh,
                                                         const int32_t* __restrict__ sorted_ids,
                                                         const float* __restrict__ sorted_w,
                                                         const int32_t* __restrict__ block_expert,
                                                         const int32_t* __restrict__ num_valid,
                                                         const int32_t* __restrict__ rows, int bm, int64_t tokens,
                                                         __nv_bfloat16* __restrict__ slots) {
  __shared__ float hs[kI];
  const int64_t row = rows ? rows[blockIdx.x] : blockIdx.x;
  if (row >= num_valid[0]) return;
  const int sid = sorted_ids[row];
  const int64_t token = sid & 0x00ffffff;
  if (token >= tokens) return;
  const int slot = sid >> 24;
  const int e = block_expert[row / bm];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int k = threadIdx.x; k < kI; k += 256) {
    const uint32_t byte = hq[row * (kI / 2) + (k >> 1)];
    const int g = k >> 5;
    const uint32_t sc = sfh[((row / bm) * (kI / 128) + (g >> 2)) * kAtomBytes + atom_offset(static_cast<int>(row % bm), g & 3)];
    hs[k] = e2m1_value((byte >> ((k & 1) * 4)) & 15u) * e8m0_value(sc);
  }
  __syncthreads();
  const float wt = sorted_w[row];
#pragma unroll 1
  for (int j = 0; j < 8; ++j) {
    const int n = blockIdx.y * 64 + warp * 8 + j;
    const int64_t wrow = static_cast<int64_t>(e) * kH + n;
    const uint4* wq = reinterpret_cast<const uint4*>(w2 + wrow * (kI / 2));
    float acc = 0.0f;
    for (int blk = lane; blk < kI / 32; blk += 32)
      acc += dot32(wq[blk], hs + blk * 32, e8m0_value(s2[wrow * (kI / 32) + blk]));
    acc = warp_sum(acc);
    if (lane == 0) slots[(token * kTopK + slot) * kH + n] = __float2bfloat16_rn(acc * wt);
  }
}

}  // namespace b200moe

extern "C" int b200moe_gemm1_simt(const uint8_t* w13, const uint8_t* w13_scale, const uint8_t* codes,
                                  const uint8_t* scales, const int32_t* sorted_ids, const int32_t* block_expert,
                                  const int32_t* num_valid, const int32_t* rows, int64_t n_rows, int64_t max_rows, int bm,
                                  int64_t tokens, uint8_t* hq, uint8_t* sfh, void* stream) {
  using namespace b200moe;
  if (!w13 || !w13_scale || !codes || !scales || !sorted_ids || !block_expert || !num_valid || !hq || !sfh)
    return B200MOE_E_ARG;
  if (bm != 16 && bm != 32 && bm != 64 && bm != 128) return B200MOE_E_ARG;
  const int64_t n = rows ? n_rows : max_rows;
  if (n <= 0) return 0;
  B200MOE_LAUNCH_PLAIN(gemm1_simt_kernel, dim3(static_cast<unsigned>(n), kI / 32), 256, 0, static_cast<cudaStream_t>(stream), w13, w13_scale, codes, scales, sorted_ids, block_expert, num_valid, rows, bm, tokens, hq, sfh);
  return 0;
}

extern "C" int b200moe_gemm2_simt(const uint8_t* w2, const uint8_t* w2_scale, const uint8_t* hq, const uint8_t* sfh,
                                  const int32_t* sorted_ids, const float* sorted_w, const int32_t* block_expert,
                                  const int32_t* num_valid, const int32_t* rows, int64_t n_rows, int64_t max_rows, int bm,
                                  int64_t tokens, void* slots_bf16, void* stream) {
  using namespace b200moe;
  if (!w2 || !w2_scale || !hq || !sfh || !sorted_ids || !sorted_w || !block_expert || !num_valid || !slots_bf16)
    return B200MOE_E_ARG;
  if (bm != 16 && bm != 32 && bm != 64 && bm != 128) return B200MOE_E_ARG;
  const int64_t n = rows ? n_rows : max_rows;
  if (n <= 0) return 0;
  B200MOE_LAUNCH_PLAIN(gemm2_simt_kernel, dim3(static_cast<unsigned>(n), kH / 64), 256, 0, static_cast<cudaStream_t>(stream), w2, w2_scale, hq, sfh, sorted_ids, sorted_w, block_expert, num_valid, rows, bm, tokens, static_cast<__nv_bfloat16*>(slots_bf16));
  return 0;
}
