// Router top-4: one warp per token, four experts per lane, four rounds of warp arg-max.
#include "common.cuh"

namespace b200moe {

// (value, id) ordering: larger value first, equal values to the lower id.
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

template <int MODE>
__global__ void __launch_bounds__(256) route_topk_kernel(const float* __restrict__ partials, int64_t stride_t,
                                                         int64_t stride_s, int splits, const float* __restrict__ bias,
                                                         int64_t tokens, int num_experts, float scale,
                                                         float* __restrict__ out_w, int32_t* __restrict__ out_ids) {
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  // lane owns experts lane, lane+32, lane+64, lane+96 (coalesced loads)
  float logit[4], score[4], choice[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = lane + 32 * j;
    float acc = 0.0f;
    if (e < num_experts) {
      const float* p = partials + t * stride_t + e;
      for (int s = 0; s < splits; ++s) acc = acc + p[s * stride_s];
    }
    logit[j] = acc;
    if (MODE == B200MOE_ROUTE_SIGMOID_BIAS) {
      score[j] = 1.0f / (1.0f + expf(-acc));
      choice[j] = score[j] + (bias ? bias[e < num_experts ? e : 0] : 0.0f);
    } else {
      score[j] = acc;
      choice[j] = acc;
    }
    if (e >= num_experts) choice[j] = -INFINITY;
  }
  float sel_score[4];
  int sel_id[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    float bs = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = lane + 32 * j;
      if (e < num_experts && better(choice[j], e, bv, bi)) { bv = choice[j]; bi = e; bs = score[j]; }
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      const float os = __shfl_xor_sync(0xffffffffu, bs, off);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; bs = os; }
    }
    if (bi == 0x7fffffff) { bi = r; bs = 0.0f; }  // nothing comparable left (NaN row): the round number
    sel_id[r] = bi;
    sel_score[r] = bs;
    if ((bi & 31) == lane) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (j == (bi >> 5)) choice[j] = -INFINITY;
    }
  }
  float w[4];
  if (MODE == B200MOE_ROUTE_SIGMOID_BIAS) {
    const float sum = ((sel_score[0] + sel_score[1]) + sel_score[2]) + sel_score[3];
#pragma unroll
    for (int r = 0; r < 4; ++r) w[r] = sel_score[r] * scale / sum;
  } else {
    float p[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) p[r] = expf(sel_score[r] - sel_score[0]);
    const float sum = ((p[0] + p[1]) + p[2]) + p[3];
#pragma unroll
    for (int r = 0; r < 4; ++r) w[r] = p[r] * scale / sum;
  }
  if (lane < 4) {
    float wv = w[0];
    int iv = sel_id[0];
#pragma unroll
    for (int r = 1; r < 4; ++r)
      if (lane == r) { wv = w[r]; iv = sel_id[r]; }
    out_w[t * 4 + lane] = wv;
    out_ids[t * 4 + lane] = iv;
  }
}

}  // namespace b200moe

extern "C" int b200moe_route_topk(const float* partials, int64_t stride_t, int64_t stride_s, int splits,
                                  const float* bias, int64_t tokens, int num_experts, int mode, float scale,
                                  float* out_w, int32_t* out_ids, void* stream) {
  using namespace b200moe;
  if (!partials || !out_w || !out_ids || tokens < 0 || splits < 1 || num_experts < 4 || num_experts > kMaxE)
    return B200MOE_E_ARG;
  if (mode != B200MOE_ROUTE_SIGMOID_BIAS && mode != B200MOE_ROUTE_SOFTMAX) return B200MOE_E_ARG;
  if (tokens == 0) return 0;
  const int warps = 8;
  const unsigned grid = static_cast<unsigned>((tokens + warps - 1) / warps);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (mode == B200MOE_ROUTE_SIGMOID_BIAS)
    route_topk_kernel<B200MOE_ROUTE_SIGMOID_BIAS><<<grid, warps * 32, 0, s>>>(partials, stride_t, stride_s, splits, bias,
                                                                             tokens, num_experts, scale, out_w, out_ids);
  else
    route_topk_kernel<B200MOE_ROUTE_SOFTMAX><<<grid, warps * 32, 0, s>>>(partials, stride_t, stride_s, splits, bias,
                                                                        tokens, num_experts, scale, out_w, out_ids);
  B200MOE_CHECK_LAUNCH();
  return 0;
}
