// Router GEMM: bf16 activations x fp32 gate -> fp32 split-K partial logits [S][T][E], consumed by the top-4 kernel, which
// adds the partials from 0.0 in split order. Products are exact in fp32 (a bf16 factor has 8 significant bits) and each
// partial is a short fp32 FMA chain, so the error per partial stays far below 2^-18 * sum|x||w| (the bound the reference
// states for its three-term bf16 split). CUDA cores: 1.6 MFLOP per token is noise next to the experts' 113 MFLOP.
#include "common.cuh"

namespace b200moe {

constexpr int kRgTokens = 16;   // tokens per CTA
constexpr int kRgK = 32;        // K elements per shared-memory tile

// What the fused form also writes, row-major: the routed experts' MXFP4 operands and (optionally) the shared expert's
// MXFP8 operands of the same rows. A shared-memory tile is 16 tokens x 32 K-elements = one quantisation block per token.
struct QuantOut {
  uint8_t* codes4;   // [T][3072]
  uint8_t* scales4;  // [T][192]
  uint8_t* codes8;   // [T][6144], may be null
  uint8_t* scales8;  // [T][192]
};

// grid (ceil(T/16), S); 256 threads: thread = (expert e = tid % 128, token half th = tid / 128 -> 8 tokens)
template <bool QUANT>
__global__ void __launch_bounds__(256) router_gemm_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const float* __restrict__ gate, int64_t tokens,
                                                          int num_experts, int k_per_split,
                                                          float* __restrict__ partials, QuantOut q) {
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
    if (QUANT) {
      // one pass over x: the tile's 16 blocks of 32 values are quantised while they sit in shared memory. Thread =
      // (token r = tid / 16, value pair c2 = tid % 16); the 16 lanes of a block share its maximum.
      const int r = tid >> 4, c2 = tid & 15;
      const float v0 = xs[r][2 * c2], v1 = xs[r][2 * c2 + 1];
      float amax = fmaxf(fabsf(v0), fabsf(v1));
#pragma unroll
      for (int m = 1; m < 16; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
      const int64_t t = t0 + r;
      if (t < tokens) {
        const int k = k0 + kk;
        const int e4 = quark_even_e8m0(amax);
        const float inv4 = __uint_as_float(static_cast<uint32_t>(254 - e4) << 23);
        q.codes4[t * (kH / 2) + (k >> 1) + c2] = static_cast<uint8_t>(cvt_e2m1x2(v0 * inv4, v1 * inv4));
        if (c2 == 0) q.scales4[t * (kH / 32) + (k >> 5)] = static_cast<uint8_t>(e4);
        if (q.codes8 != nullptr) {
          const int e8 = mxfp8_scale(amax);
          const float inv8 = __uint_as_float(static_cast<uint32_t>(254 - e8) << 23);
          *reinterpret_cast<uint16_t*>(q.codes8 + t * kH + k + 2 * c2) = static_cast<uint16_t>(cvt_e4m3x2(v0 * inv8, v1 * inv8));
          if (c2 == 0) q.scales8[t * (kH / 32) + (k >> 5)] = static_cast<uint8_t>(e8);
        }
      }
    }
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
  B200MOE_LAUNCH(router_gemm_kernel<false>, grid, 256, 0, static_cast<cudaStream_t>(stream),
                 static_cast<const __nv_bfloat16*>(x_bf16), gate, tokens, num_experts, kH / splits, partials, QuantOut{});
  return 0;
}

extern "C" int b200moe_router_gemm_quant(const void* x_bf16, const float* gate, int64_t tokens, int num_experts, int splits,
                                         float* partials, uint8_t* codes4, uint8_t* scales4, uint8_t* codes8,
                                         uint8_t* scales8, void* stream) {
  using namespace b200moe;
  if (!x_bf16 || !gate || !partials || !codes4 || !scales4 || tokens < 0 || num_experts < 1 || num_experts > kMaxE)
    return B200MOE_E_ARG;
  if ((codes8 != nullptr) != (scales8 != nullptr)) return B200MOE_E_ARG;
  if (splits < 1 || kH % splits || (kH / splits) % kRgK) return B200MOE_E_ARG;
  if (reinterpret_cast<uintptr_t>(codes8) & 1) return B200MOE_E_ALIGN;
  if (tokens == 0) return 0;
  const dim3 grid(static_cast<unsigned>((tokens + kRgTokens - 1) / kRgTokens), static_cast<unsigned>(splits));
  const QuantOut q{codes4, scales4, codes8, scales8};
  B200MOE_LAUNCH(router_gemm_kernel<true>, grid, 256, 0, static_cast<cudaStream_t>(stream),
                 static_cast<const __nv_bfloat16*>(x_bf16), gate, tokens, num_experts, kH / splits, partials, q);
  return 0;
}
