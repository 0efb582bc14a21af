// Router GEMM: bf16 activations x fp32 gate -> fp32 split-K partial logits [S][T][E], consumed by the top-4 kernel, which
// adds the partials from 0.0 in split order. Products are exact in fp32 (a bf16 factor has 8 significant bits) and each
// partial is a short fp32 FMA chain, so the error per partial stays far below 2^-18 * sum|x||w| (the bound the reference
// states for its three-term bf16 split). CUDA cores: 1.6 MFLOP per token is noise next to the experts' 113 MFLOP.
#include "common.cuh"

namespace b200moe {

constexpr int kRgTokens = 16;   // tokens per CTA
constexpr int kRgK = 32;        // K elements per shared-memory tile

// grid (ceil(T/16), S); 256 threads: thread = (expert e = tid % 128, token half th = tid / 128 -> 8 tokens)
__global__ void __launch_bounds__(256) router_gemm_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const float* __restrict__ gate, int64_t tokens,
                                                          int num_experts, int k_per_split,
                                                          float* __restrict__ partials) {
  __shared__ float ws[kMaxE][kRgK + 1];
  __shared__ float xs[kRgTokens][kRgK];
  pdl_enter(x, gate);
  const int tid = threadIdx.x, e = tid & 127, th = tid >> 7;
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * kRgTokens;
  const int k0 = blockIdx.y * k_per_split;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  for (int kk = 0; kk < k_per_split; kk += kRgK) {
    // gate tile: 128 rows x 32 floats, a warp reads one row's 128 bytes
    for (int i = tid; i < kMaxE * kRgK; i += 256) {
      const int r = i >> 5, c = i & 31;
      ws[r][c] = r < num_experts ? gate[static_cast<int64_t>(r) * kH + k0 + kk + c] : 0.0f;
    }
    for (int i = tid; i < kRgTokens * kRgK; i += 256) {
      const int r = i >> 5, c = i & 31;
      xs[r][c] = t0 + r < tokens ? __bfloat162float(x[(t0 + r) * kH + k0 + kk + c]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < kRgK; ++c) {
      const float wv = ws[e][c];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(xs[th * 8 + j][c], wv, acc[j]);
    }
    __syncthreads();
  }
  if (e < num_experts) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t t = t0 + th * 8 + j;
      if (t < tokens) partials[(static_cast<int64_t>(blockIdx.y) * tokens + t) * num_experts + e] = acc[j];
    }
  }
}

}  // namespace b200moe

extern "C" int b200moe_router_splits(int64_t tokens) { return tokens <= 2048 ? 16 : 4; }

extern "C" int b200moe_router_gemm(const void* x_bf16, const float* gate, int64_t tokens, int num_experts, int splits,
                                   float* partials, void* stream) {
  using namespace b200moe;
  if (!x_bf16 || !gate || !partials || tokens < 0 || num_experts < 1 || num_experts > kMaxE) return B200MOE_E_ARG;
  if (splits < 1 || kH % splits || (kH / splits) % kRgK) return B200MOE_E_ARG;
  if (tokens == 0) return 0;
  const dim3 grid(static_cast<unsigned>((tokens + kRgTokens - 1) / kRgTokens), static_cast<unsigned>(splits));
  B200MOE_LAUNCH(router_gemm_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream),
                 static_cast<const __nv_bfloat16*>(x_bf16), gate, tokens, num_experts, kH / splits, partials);
  return 0;
}
