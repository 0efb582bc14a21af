// Routing sort: a stable counting sort of the 4T (token, slot) pairs by expert with per-expert padding to bm rows.
// Chunks of 1024 pairs, one CTA each. Counts are order-free; placement ranks come from warp match/popc and fixed-order
// prefix sums, so the row order inside an expert is the pair order and the result is the same on every run.
#include "common.cuh"

namespace b200moe {

constexpr int kChunk = 1024;

__global__ void __launch_bounds__(kChunk) permute_count_kernel(const int32_t* __restrict__ ids, int64_t pairs,
                                                               int num_experts, int32_t* __restrict__ cta_counts) {
  __shared__ int hist[kMaxE];
  if (threadIdx.x < kMaxE) hist[threadIdx.x] = 0;
  __syncthreads();
  const int64_t q = static_cast<int64_t>(blockIdx.x) * kChunk + threadIdx.x;
  if (q < pairs) {
    const int e = ids[q];
    if (e >= 0 && e < num_experts) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  if (threadIdx.x < num_experts) cta_counts[static_cast<int64_t>(blockIdx.x) * num_experts + threadIdx.x] = hist[threadIdx.x];
}

__global__ void __launch_bounds__(kChunk) permute_place_kernel(const int32_t* __restrict__ ids,
                                                               const float* __restrict__ w, int64_t tokens,
                                                               int num_experts, int bm,
                                                               const int32_t* __restrict__ cta_counts,
                                                               int32_t* __restrict__ sorted_ids,
                                                               float* __restrict__ sorted_w,
                                                               int32_t* __restrict__ block_expert,
                                                               int32_t* __restrict__ num_valid) {
  __shared__ int total[kMaxE];       // pairs per expert over the whole call
  __shared__ int base[kMaxE];        // pairs of this expert in earlier chunks
  __shared__ int start[kMaxE + 1];   // first padded row of each expert
  __shared__ int warp_cnt[32][kMaxE + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t pairs = tokens * kTopK;
  const int64_t q = static_cast<int64_t>(blockIdx.x) * kChunk + tid;
  int e = -1;
  if (q < pairs) {
    e = ids[q];
    if (e < 0 || e >= num_experts) e = -1;
  }
  for (int i = tid; i < 32 * (kMaxE + 1); i += kChunk) (&warp_cnt[0][0])[i] = 0;
  if (tid < kMaxE) { total[tid] = 0; base[tid] = 0; }
  __syncthreads();
  // rank inside the warp, and the warp's count per expert
  const unsigned live = __ballot_sync(0xffffffffu, e >= 0);
  int rank = 0;
  if (e >= 0) {
    const unsigned peers = __match_any_sync(live, e);
    rank = __popc(peers & ((1u << lane) - 1u));
    if (rank == 0) warp_cnt[warp][e] = __popc(peers);
  }
  if (cta_counts == nullptr) {
    __syncthreads();  // single chunk: the totals are this chunk's counts
    if (tid < num_experts) {
      int t = 0;
      for (int wi = 0; wi < 32; ++wi) t += warp_cnt[wi][tid];
      total[tid] = t;
    }
  } else if (tid < num_experts) {
    int t = 0, b = 0;
    for (unsigned c = 0; c < gridDim.x; ++c) {
      const int n = cta_counts[static_cast<int64_t>(c) * num_experts + tid];
      if (c < blockIdx.x) b += n;
      t += n;
    }
    total[tid] = t;
    base[tid] = b;
  }
  __syncthreads();
  if (tid < num_experts) {  // exclusive prefix over the warps of this chunk, in warp order
    int run = 0;
    for (int wi = 0; wi < 32; ++wi) {
      const int n = warp_cnt[wi][tid];
      warp_cnt[wi][tid] = run;
      run += n;
    }
  }
  if (tid == 0) {
    int run = 0, last = 0;
    for (int x = 0; x < num_experts; ++x) {
      start[x] = run;
      if (total[x] > 0) last = run;
      run += (total[x] + bm - 1) / bm * bm;
    }
    start[num_experts] = run;
    if (blockIdx.x == 0) { num_valid[0] = run; num_valid[1] = last; }
  }
  __syncthreads();
  if (e >= 0) {
    const int pos = start[e] + base[e] + warp_cnt[warp][e] + rank;
    const int token = static_cast<int>(q >> 2), slot = static_cast<int>(q & 3);
    sorted_ids[pos] = token | (slot << 24);
    sorted_w[pos] = w[q];
  }
  // padding rows and the block -> expert list, experts dealt round-robin to the chunks
  for (int x = blockIdx.x; x < num_experts; x += gridDim.x) {
    const int first = start[x], live_rows = total[x], padded = start[x + 1] - first;
    for (int r = live_rows + tid; r < padded; r += kChunk) {
      sorted_ids[first + r] = static_cast<int>(tokens);
      sorted_w[first + r] = 0.0f;
    }
    for (int b = tid; b < padded / bm; b += kChunk) block_expert[first / bm + b] = x;
  }
}

}  // namespace b200moe

extern "C" size_t b200moe_permute_scratch_bytes(int64_t tokens, int num_experts) {
  const int64_t chunks = (tokens * b200moe::kTopK + b200moe::kChunk - 1) / b200moe::kChunk;
  return chunks > 1 ? static_cast<size_t>(chunks) * num_experts * sizeof(int32_t) : 0;
}

extern "C" int64_t b200moe_max_sorted_rows(int64_t tokens, int bm, int num_experts) {
  const int64_t pairs = tokens * b200moe::kTopK;
  const int64_t ex = pairs < num_experts ? pairs : num_experts;
  return (pairs + ex * (bm - 1) + bm - 1) / bm * bm;
}

extern "C" int b200moe_block_rows(int64_t tokens) {
  if (tokens <= 128) return 16;
  if (tokens <= 512) return 32;
  if (tokens <= 1024) return 64;
  return 128;
}

extern "C" int b200moe_permute(const int32_t* ids, const float* w, int64_t tokens, int num_experts, int bm,
                               int32_t* sorted_ids, float* sorted_w, int32_t* block_expert, int32_t* num_valid,
                               int32_t* scratch, void* stream) {
  using namespace b200moe;
  if (!ids || !w || !sorted_ids || !sorted_w || !block_expert || !num_valid) return B200MOE_E_ARG;
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS || num_experts < 1 || num_experts > kMaxE) return B200MOE_E_ARG;
  if (bm != 16 && bm != 32 && bm != 64 && bm != 128) return B200MOE_E_ARG;
  const int64_t pairs = tokens * kTopK;
  const unsigned chunks = static_cast<unsigned>((pairs + kChunk - 1) / kChunk);
  if (chunks > 1 && !scratch) return B200MOE_E_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (chunks > 1) {
    permute_count_kernel<<<chunks, kChunk, 0, s>>>(ids, pairs, num_experts, scratch);
    B200MOE_CHECK_LAUNCH();
  }
  permute_place_kernel<<<chunks, kChunk, 0, s>>>(ids, w, tokens, num_experts, bm, chunks > 1 ? scratch : nullptr,
                                                 sorted_ids, sorted_w, block_expert, num_valid);
  B200MOE_CHECK_LAUNCH();
  return 0;
}
