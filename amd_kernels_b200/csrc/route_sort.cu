// Router top-4 and the routing sort (a stable counting sort of the 4T (token, slot) pairs by expert with per-expert
// padding to bm rows). Up to 32 tokens both run in ONE single-CTA kernel; above that the router is its own grid and the
// sort runs as a count pass (above 256 tokens) and a placement pass over 1024-pair chunks.
//
// Determinism: counts are order-free; placement ranks come from warp match/popc and fixed-order prefix sums, so the row
// order inside an expert is the pair order 4*token+slot on every run.
#include <mutex>

#include "common.cuh"

namespace b200moe {

constexpr int kChunk = 1024;
constexpr int kFusedRouteTokens = 32;  // up to here the single-CTA kernel routes one token per warp and sorts

// (value, id) ordering: larger value first, equal values to the lower id.
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

// One warp routes one token. Lane owns experts lane, lane+32, lane+64, lane+96. Every lane returns the 4 picks.
template <int MODE>
__device__ __forceinline__ void route_token(const float* __restrict__ row, int64_t stride_s, int splits,
                                            const float* __restrict__ bias, int num_experts, float scale, int lane,
                                            float (&w)[4], int (&sel_id)[4]) {
  float score[4], choice[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = lane + 32 * j;
    float acc = 0.0f;
    if (e < num_experts)
      for (int s = 0; s < splits; ++s) acc = acc + row[s * stride_s + e];
    if (MODE == B200MOE_ROUTE_SIGMOID_BIAS) {
      score[j] = 1.0f / (1.0f + expf(-acc));
      choice[j] = score[j] + (bias && e < num_experts ? bias[e] : 0.0f);
    } else {
      score[j] = acc;
      choice[j] = acc;
    }
    if (e >= num_experts) choice[j] = -INFINITY;
  }
  float sel_score[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    float bv = -INFINITY, bs = 0.0f;
    int bi = 0x7fffffff;
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
    if (bi == 0x7fffffff) { bi = r; bs = 0.0f; }  // nothing comparable left (a NaN row): the round number
    sel_id[r] = bi;
    sel_score[r] = bs;
    if ((bi & 31) == lane) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (j == (bi >> 5)) choice[j] = -INFINITY;
    }
  }
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
}

template <int MODE>
__global__ void __launch_bounds__(256) route_topk_kernel(const float* __restrict__ partials, int64_t stride_t,
                                                         int64_t stride_s, int splits, const float* __restrict__ bias,
                                                         int64_t tokens, int num_experts, float scale,
                                                         float* __restrict__ out_w, int32_t* __restrict__ out_ids) {
  pdl_enter(partials, bias);
  const int lane = threadIdx.x & 31;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  float w[4];
  int id[4];
  route_token<MODE>(partials + t * stride_t, stride_s, splits, bias, num_experts, scale, lane, w, id);
  if (lane < 4) {
    float wv = w[0];
    int iv = id[0];
#pragma unroll
    for (int r = 1; r < 4; ++r)
      if (lane == r) { wv = w[r]; iv = id[r]; }
    out_w[t * 4 + lane] = wv;
    out_ids[t * 4 + lane] = iv;
  }
}

// `limit` (may be null): a device count of the pairs that are live; pairs from there on are ignored whatever their id (the
// expert-parallel receive buffers are sorted at full capacity without the arrived count ever reaching the host).
__global__ void __launch_bounds__(kChunk) permute_count_kernel(const int32_t* __restrict__ ids, int64_t pairs,
                                                               int num_experts, int32_t* __restrict__ cta_counts,
                                                               const int32_t* __restrict__ limit) {
  pdl_enter(ids, limit);
  __shared__ int hist[kMaxE];
  if (threadIdx.x < kMaxE) hist[threadIdx.x] = 0;
  __syncthreads();
  if (limit != nullptr) pairs = min(pairs, static_cast<int64_t>(__ldcg(limit)));
  const int64_t q = static_cast<int64_t>(blockIdx.x) * kChunk + threadIdx.x;
  if (q < pairs) {
    const int e = __ldcg(ids + q);
    if (e >= 0 && e < num_experts) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  if (threadIdx.x < num_experts) cta_counts[static_cast<int64_t>(blockIdx.x) * num_experts + threadIdx.x] = hist[threadIdx.x];
}

struct SortShared {
  int total[kMaxE];        // pairs per expert over the whole call
  int base[kMaxE];         // pairs of this expert in earlier chunks
  int start[kMaxE + 4];    // first padded row of each expert, [num_experts] = padded total
  int warp_cnt[32][kMaxE + 1];
};

// The placement of one 1024-pair chunk. e = this thread's expert (or -1), wv its routing weight, q its pair index.
__device__ __forceinline__ void place_chunk(SortShared& sh, int e, float wv, int64_t q, int64_t tokens, int num_experts,
                                            int bm_shift, const int32_t* __restrict__ cta_counts,
                                            int32_t* __restrict__ sorted_ids, float* __restrict__ sorted_w,
                                            int32_t* __restrict__ block_expert, int32_t* __restrict__ num_valid,
                                            int* pos_out = nullptr) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bm = 1 << bm_shift;
  for (int i = tid; i < 32 * (kMaxE + 1); i += kChunk) (&sh.warp_cnt[0][0])[i] = 0;
  if (tid < kMaxE) { sh.total[tid] = 0; sh.base[tid] = 0; }
  __syncthreads();
  // rank inside the warp, and the warp's count per expert
  const unsigned live = __ballot_sync(0xffffffffu, e >= 0);
  int rank = 0;
  if (e >= 0) {
    const unsigned peers = __match_any_sync(live, e);
    rank = __popc(peers & ((1u << lane) - 1u));
    if (rank == 0) sh.warp_cnt[warp][e] = __popc(peers);
  }
  __syncthreads();
  if (tid < num_experts) {
    // exclusive prefix over the warps of this chunk in warp order; totals and the base of earlier chunks
    int run = 0;
#pragma unroll 8
    for (int wi = 0; wi < 32; ++wi) {
      const int n = sh.warp_cnt[wi][tid];
      sh.warp_cnt[wi][tid] = run;
      run += n;
    }
    int t = run, b = 0;
    if (cta_counts != nullptr) {
      t = 0;
      for (unsigned c = 0; c < gridDim.x; ++c) {
        const int n = __ldcg(cta_counts + static_cast<int64_t>(c) * num_experts + tid);
        if (c < blockIdx.x) b += n;
        t += n;
      }
    }
    sh.total[tid] = t;
    sh.base[tid] = b;
  }
  __syncthreads();
  if (warp == 0) {
    // padded sizes and their exclusive scan over the experts: lane owns experts 4*lane .. 4*lane+3
    int pad[4], sum = 0, last = -1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int x = 4 * lane + j;
      const int t = x < num_experts ? sh.total[x] : 0;
      pad[j] = ((t + bm - 1) >> bm_shift) << bm_shift;
      sum += pad[j];
      if (t > 0) last = x;
    }
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    int run = incl - sum;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sh.start[4 * lane + j] = run;
      run += pad[j];
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, off));
    const int grand = __shfl_sync(0xffffffffu, incl, 31);
    __syncwarp();
    if (lane == 0) {
      sh.start[num_experts] = grand;  // experts beyond num_experts have zero size, so start[num_experts] == total
      if (blockIdx.x == 0) {
        num_valid[0] = grand;
        num_valid[1] = last >= 0 ? sh.start[last] : 0;
      }
    }
  }
  __syncthreads();
  if (e >= 0) {
    const int pos = sh.start[e] + sh.base[e] + sh.warp_cnt[warp][e] + rank;
    sorted_ids[pos] = static_cast<int>(q >> 2) | (static_cast<int>(q & 3) << 24);
    sorted_w[pos] = wv;
    if (pos_out != nullptr) *pos_out = pos;
  }
  // padding rows and the block -> expert list: experts dealt round-robin to the chunks, then to the warps
  for (int x = blockIdx.x + warp * gridDim.x; x < num_experts; x += 32 * gridDim.x) {
    const int first = sh.start[x], live_rows = sh.total[x];
    const int padded = (((live_rows + bm - 1) >> bm_shift) << bm_shift);
    for (int r = live_rows + lane; r < padded; r += 32) {
      sorted_ids[first + r] = static_cast<int>(tokens);
      sorted_w[first + r] = 0.0f;
    }
    for (int b = lane; b < (padded >> bm_shift); b += 32) block_expert[(first >> bm_shift) + b] = x;
  }
}

__global__ void __launch_bounds__(kChunk) permute_place_kernel(const int32_t* __restrict__ ids,
                                                               const float* __restrict__ w, int64_t tokens,
                                                               int num_experts, int bm_shift,
                                                               const int32_t* __restrict__ cta_counts,
                                                               int32_t* __restrict__ sorted_ids,
                                                               float* __restrict__ sorted_w,
                                                               int32_t* __restrict__ block_expert,
                                                               int32_t* __restrict__ num_valid,
                                                               const int32_t* __restrict__ limit) {
  pdl_enter(ids, w, cta_counts, limit);
  __shared__ SortShared sh;
  int64_t pairs = tokens * kTopK;
  if (limit != nullptr) pairs = min(pairs, static_cast<int64_t>(__ldcg(limit)));
  const int64_t q = static_cast<int64_t>(blockIdx.x) * kChunk + threadIdx.x;
  int e = -1;
  float wv = 0.0f;
  if (q < pairs) {
    e = __ldcg(ids + q);
    wv = __ldcg(w + q);
    if (e < 0 || e >= num_experts) e = -1;
  }
  place_chunk(sh, e, wv, q, tokens, num_experts, bm_shift, cta_counts, sorted_ids, sorted_w, block_expert, num_valid);
}

// Up to 32 tokens: routing and the sort in one CTA. Warp w routes tokens w, w+32, ... `logits` are plain logits
// (splits = 1) or split-K partials added in split order (row t at t*stride_t, split s at s*stride_s).
template <int MODE>
__global__ void __launch_bounds__(kChunk) route_sort_kernel(const float* __restrict__ logits, int64_t stride_t,
                                                            int64_t stride_s, int splits,
                                                            const float* __restrict__ bias, int tokens,
                                                            int num_experts, float scale, int bm_shift,
                                                            float* __restrict__ out_w, int32_t* __restrict__ out_ids,
                                                            int32_t* __restrict__ sorted_ids,
                                                            float* __restrict__ sorted_w,
                                                            int32_t* __restrict__ block_expert,
                                                            int32_t* __restrict__ num_valid) {
  pdl_enter(logits, bias);
  __shared__ SortShared sh;
  __shared__ int s_ids[kChunk];
  __shared__ float s_w[kChunk];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t = warp; t < tokens; t += 32) {
    float w[4];
    int id[4];
    route_token<MODE>(logits + static_cast<int64_t>(t) * stride_t, stride_s, splits, bias, num_experts, scale, lane, w, id);
    if (lane < 4) {
      float wv = w[0];
      int iv = id[0];
#pragma unroll
      for (int r = 1; r < 4; ++r)
        if (lane == r) { wv = w[r]; iv = id[r]; }
      s_ids[t * 4 + lane] = iv;
      s_w[t * 4 + lane] = wv;
      out_w[t * 4 + lane] = wv;
      out_ids[t * 4 + lane] = iv;
    }
  }
  __syncthreads();
  const int q = threadIdx.x;
  int e = -1;
  float wv = 0.0f;
  if (q < tokens * kTopK) { e = s_ids[q]; wv = s_w[q]; }
  place_chunk(sh, e, wv, q, tokens, num_experts, bm_shift, nullptr, sorted_ids, sorted_w, block_expert, num_valid);
}

// Up to 32 tokens, ONE launch prepares the grouped GEMMs' input: every CTA of a small grid routes all tokens and sorts all
// pairs by itself (a few microseconds of redundant work, and identical stores of the same values to the routing tables, in
// exchange for a launch and a grid-wide dependency less), then the CTAs share the sorted rows among them: four rows at a
// time per CTA, 256 threads each, quantised from the bf16 row (GATHER false) or copied from row-major quantised rows
// (GATHER true: the router inside the call has quantised the tokens already). CTA 0 also zeroes `done`.
constexpr int kPrepMaxRows = 2048;  // 32 tokens x 4 pairs, every pair alone in a 16-row block
template <int MODE, bool GATHER>
__global__ void __launch_bounds__(kChunk) prep_small_kernel(const float* __restrict__ logits, int64_t stride_t,
                                                            int64_t stride_s, int splits, const float* __restrict__ bias,
                                                            int tokens, int num_experts, float scale, int bm_shift,
                                                            float* __restrict__ out_w, int32_t* __restrict__ out_ids,
                                                            int32_t* __restrict__ sorted_ids, float* __restrict__ sorted_w,
                                                            int32_t* __restrict__ block_expert,
                                                            int32_t* __restrict__ num_valid, const uint4* __restrict__ x,
                                                            const uint8_t* __restrict__ q4, const uint8_t* __restrict__ s4,
                                                            uint8_t* __restrict__ xq_sorted, uint8_t* __restrict__ sfx,
                                                            int32_t* __restrict__ done, int n_done) {
  pdl_enter(logits, bias, x, q4, s4);
  __shared__ SortShared sh;
  __shared__ int s_ids[kTopK * kFusedRouteTokens];
  __shared__ float s_w[kTopK * kFusedRouteTokens];
  __shared__ int16_t s_token[kPrepMaxRows];  // token of a sorted row, -1 for a padding row
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (blockIdx.x == 0)
    for (int z = threadIdx.x; z < n_done; z += kChunk) done[z] = 0;
  for (int i = threadIdx.x; i < kPrepMaxRows; i += kChunk) s_token[i] = -1;
  if (warp < tokens) {
    float w[4];
    int id[4];
    route_token<MODE>(logits + static_cast<int64_t>(warp) * stride_t, stride_s, splits, bias, num_experts, scale, lane, w, id);
    if (lane < 4) {
      float wv = w[0];
      int iv = id[0];
#pragma unroll
      for (int r = 1; r < 4; ++r)
        if (lane == r) { wv = w[r]; iv = id[r]; }
      s_ids[warp * 4 + lane] = iv;
      s_w[warp * 4 + lane] = wv;
      if (blockIdx.x == 0) {
        out_w[warp * 4 + lane] = wv;
        out_ids[warp * 4 + lane] = iv;
      }
    }
  }
  __syncthreads();
  const int q = threadIdx.x;
  int e = -1, pos = -1;
  float wv = 0.0f;
  if (q < tokens * kTopK) { e = s_ids[q]; wv = s_w[q]; }
  place_chunk(sh, e, wv, q, tokens, num_experts, bm_shift, nullptr, sorted_ids, sorted_w, block_expert, num_valid, &pos);
  if (pos >= 0 && pos < kPrepMaxRows) s_token[pos] = static_cast<int16_t>(q >> 2);
  __syncthreads();
  const int rows = min(sh.start[num_experts], kPrepMaxRows);
  const int sub = threadIdx.x >> 8, t = threadIdx.x & 255;  // four rows at a time per CTA
  for (int row = blockIdx.x * 4 + sub; row < rows; row += gridDim.x * 4) {
    const int token = s_token[row];
    uint32_t* dst = reinterpret_cast<uint32_t*>(xq_sorted + static_cast<int64_t>(row) * (kH / 2));
    const int r = row & ((1 << bm_shift) - 1);
    uint8_t* sdst = sfx + static_cast<int64_t>(row >> bm_shift) * (kH / 128) * kAtomBytes + atom_offset(r, 0);
    if (token < 0) quant_row_to_atoms(nullptr, dst, sdst, t);
    else if (GATHER) copy_row_to_atoms(q4 + static_cast<int64_t>(token) * (kH / 2), s4 + static_cast<int64_t>(token) * (kH / 32), dst, sdst, t);
    else quant_row_to_atoms(x + static_cast<int64_t>(token) * (kH / 8), dst, sdst, t);
  }
}

// Expert-parallel send plan, part 1: the destination rank of every (token, slot) pair and the number of pairs per rank.
// One CTA; integer counts, so the result does not depend on the order of the atomics.
__global__ void __launch_bounds__(kChunk) ep_dest_kernel(const int32_t* __restrict__ ids, int64_t pairs, int world,
                                                         int experts_per_rank, int interleaved,
                                                         int32_t* __restrict__ dest, int64_t* __restrict__ counts) {
  pdl_enter(ids);
  __shared__ int hist[8];
  if (threadIdx.x < 8) hist[threadIdx.x] = 0;
  __syncthreads();
  for (int64_t q = threadIdx.x; q < pairs; q += kChunk) {
    const int e = __ldcg(ids + q);
    int d = interleaved ? e % world : e / experts_per_rank;
    if (e < 0 || d >= world) d = -1;
    dest[q] = d;
    if (d >= 0) atomicAdd(&hist[d], 1);
  }
  __syncthreads();
  if (threadIdx.x < world) counts[threadIdx.x] = hist[threadIdx.x];
}

// Part 2, after the ranks exchanged their counts (matrix[s][d] = pairs rank s sends to rank d): where this rank's segment
// starts in its own send order and in every destination's receive buffers, and how many pairs it receives.
__global__ void ep_offsets_kernel(const int64_t* __restrict__ matrix, int world, int rank, int32_t* __restrict__ seg_start,
                                  int64_t* __restrict__ dst_base, int32_t* __restrict__ recv_pairs) {
  pdl_enter(matrix);
  const int d = threadIdx.x;
  if (d < world) {
    int64_t before = 0, base = 0;
    for (int k = 0; k < d; ++k) before += __ldcg(matrix + rank * world + k);
    for (int s = 0; s < rank; ++s) base += __ldcg(matrix + s * world + d);
    seg_start[d] = static_cast<int32_t>(before);
    dst_base[d] = base;
  }
  if (d == 0) {
    int64_t n = 0;
    for (int s = 0; s < world; ++s) n += __ldcg(matrix + s * world + rank);
    *recv_pairs = static_cast<int32_t>(n);
  }
}

// The sorted row blocks split into `chunks` runs of (nearly) equal length: ranges[i] = {first block, one past the last} of
// run i. The count of blocks is on the device only (num_valid), hence a kernel.
__global__ void block_chunks_kernel(const int32_t* __restrict__ num_valid, int bm, int chunks, int32_t* __restrict__ ranges) {
  pdl_enter(num_valid);
  const int i = threadIdx.x;
  if (i < chunks) {
    const int64_t n = max(0, __ldcg(num_valid)) / bm;
    ranges[2 * i] = static_cast<int32_t>(n * i / chunks);
    ranges[2 * i + 1] = static_cast<int32_t>(n * (i + 1) / chunks);
  }
}

// bm = 1 (no padding) serves the expert-parallel send order: pairs grouped by destination rank
static int shift_of(int bm) { return bm == 1 ? 0 : bm == 16 ? 4 : bm == 32 ? 5 : bm == 64 ? 6 : bm == 128 ? 7 : -1; }

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
    B200MOE_LAUNCH((route_topk_kernel<B200MOE_ROUTE_SIGMOID_BIAS>), grid, warps * 32, 0, s, partials, stride_t, stride_s,
                   splits, bias, tokens, num_experts, scale, out_w, out_ids);
  else
    B200MOE_LAUNCH((route_topk_kernel<B200MOE_ROUTE_SOFTMAX>), grid, warps * 32, 0, s, partials, stride_t, stride_s, splits,
                   bias, tokens, num_experts, scale, out_w, out_ids);
  return 0;
}

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
  // by measurement (layer time, graph replays): 16-row blocks to 480 tokens, 32-row blocks to 512, from there the 128-row
  // path (row quantiser + GEMM1 that gathers its rows + 256 weight rows per MMA), which at 1024 / 1400 / 1728 tokens takes
  // 196 / 208 / 211 us against 232 / 248 / 265 us with 32- and 64-row blocks (600 tokens: 190 against 194; 400: 187 against
  // 182). The 64-row kernels stay in the library for callers that sort with that block height themselves.
  if (tokens <= 480) return 16;
  if (tokens <= 512) return 32;
  return 128;
}

extern "C" int b200moe_permute(const int32_t* ids, const float* w, int64_t tokens, int num_experts, int bm,
                               int32_t* sorted_ids, float* sorted_w, int32_t* block_expert, int32_t* num_valid,
                               int32_t* scratch, void* stream) {
  return b200moe_permute_live(ids, w, tokens, num_experts, bm, nullptr, sorted_ids, sorted_w, block_expert, num_valid, scratch,
                              stream);
}

extern "C" int b200moe_permute_live(const int32_t* ids, const float* w, int64_t tokens, int num_experts, int bm,
                                    const int32_t* live_pairs, int32_t* sorted_ids, float* sorted_w, int32_t* block_expert,
                                    int32_t* num_valid, int32_t* scratch, void* stream) {
  using namespace b200moe;
  if (!ids || !w || !sorted_ids || !sorted_w || !block_expert || !num_valid) return B200MOE_E_ARG;
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS || num_experts < 1 || num_experts > kMaxE) return B200MOE_E_ARG;
  const int shift = shift_of(bm);
  if (shift < 0) return B200MOE_E_ARG;
  const int64_t pairs = tokens * kTopK;
  const unsigned chunks = static_cast<unsigned>((pairs + kChunk - 1) / kChunk);
  if (chunks > 1 && !scratch) return B200MOE_E_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (chunks > 1) {
    B200MOE_LAUNCH(permute_count_kernel, chunks, kChunk, 0, s, ids, pairs, num_experts, scratch, live_pairs);
  }
  B200MOE_LAUNCH(permute_place_kernel, chunks, kChunk, 0, s, ids, w, tokens, num_experts, shift, chunks > 1 ? scratch : nullptr, sorted_ids, sorted_w, block_expert, num_valid, live_pairs);
  return 0;
}

extern "C" int b200moe_route_sort_partials(const float* partials, int64_t stride_t, int64_t stride_s, int splits,
                                           const float* bias, int64_t tokens, int num_experts, int mode, float scale,
                                           int bm, float* out_w, int32_t* out_ids, int32_t* sorted_ids, float* sorted_w,
                                           int32_t* block_expert, int32_t* num_valid, int32_t* scratch, void* stream) {
  using namespace b200moe;
  if (!partials || !out_w || !out_ids || !sorted_ids || !sorted_w || !block_expert || !num_valid || splits < 1)
    return B200MOE_E_ARG;
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS || num_experts < 4 || num_experts > kMaxE) return B200MOE_E_ARG;
  if (mode != B200MOE_ROUTE_SIGMOID_BIAS && mode != B200MOE_ROUTE_SOFTMAX) return B200MOE_E_ARG;
  const int shift = shift_of(bm);
  if (shift < 0) return B200MOE_E_ARG;
  if (tokens > kFusedRouteTokens) {  // many tokens: route on many SMs first, then sort
    int r = b200moe_route_topk(partials, stride_t, stride_s, splits, bias, tokens, num_experts, mode, scale, out_w,
                               out_ids, stream);
    if (r) return r;
    return b200moe_permute(out_ids, out_w, tokens, num_experts, bm, sorted_ids, sorted_w, block_expert, num_valid, scratch,
                           stream);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (mode == B200MOE_ROUTE_SIGMOID_BIAS)
    B200MOE_LAUNCH((route_sort_kernel<B200MOE_ROUTE_SIGMOID_BIAS>), 1, kChunk, 0, s, partials, stride_t, stride_s, splits,
                   bias, static_cast<int>(tokens), num_experts, scale, shift, out_w, out_ids, sorted_ids, sorted_w,
                   block_expert, num_valid);
  else
    B200MOE_LAUNCH((route_sort_kernel<B200MOE_ROUTE_SOFTMAX>), 1, kChunk, 0, s, partials, stride_t, stride_s, splits, bias,
                   static_cast<int>(tokens), num_experts, scale, shift, out_w, out_ids, sorted_ids, sorted_w, block_expert,
                   num_valid);
  return 0;
}

extern "C" int b200moe_route_sort(const float* logits, const float* bias, int64_t tokens, int num_experts, int mode,
                                  float scale, int bm, float* out_w, int32_t* out_ids, int32_t* sorted_ids,
                                  float* sorted_w, int32_t* block_expert, int32_t* num_valid, int32_t* scratch,
                                  void* stream) {
  return b200moe_route_sort_partials(logits, num_experts, 0, 1, bias, tokens, num_experts, mode, scale, bm, out_w, out_ids,
                                     sorted_ids, sorted_w, block_expert, num_valid, scratch, stream);
}

extern "C" int b200moe_ep_dest(const int32_t* ids, int64_t tokens, int world, int experts_per_rank, int interleaved,
                               int32_t* dest, int64_t* counts, void* stream) {
  using namespace b200moe;
  if (!ids || !dest || !counts || tokens < 1 || tokens > B200MOE_MAX_TOKENS || world < 1 || world > 8 || experts_per_rank < 1)
    return B200MOE_E_ARG;
  B200MOE_LAUNCH(ep_dest_kernel, 1, kChunk, 0, static_cast<cudaStream_t>(stream), ids, tokens * kTopK, world, experts_per_rank,
                 interleaved, dest, counts);
  return 0;
}

extern "C" int b200moe_ep_offsets(const int64_t* matrix, int world, int rank, int32_t* seg_start, int64_t* dst_base,
                                  int32_t* recv_pairs, void* stream) {
  using namespace b200moe;
  if (!matrix || !seg_start || !dst_base || !recv_pairs || world < 1 || world > 8 || rank < 0 || rank >= world)
    return B200MOE_E_ARG;
  B200MOE_LAUNCH(ep_offsets_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), matrix, world, rank, seg_start, dst_base,
                 recv_pairs);
  return 0;
}

extern "C" int b200moe_block_chunks(const int32_t* num_valid, int bm, int chunks, int32_t* ranges, void* stream) {
  using namespace b200moe;
  if (!num_valid || !ranges || chunks < 1 || chunks > 32 || (bm != 16 && bm != 32 && bm != 64 && bm != 128)) return B200MOE_E_ARG;
  B200MOE_LAUNCH(block_chunks_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), num_valid, bm, chunks, ranges);
  return 0;
}

// Routing, sort and the gather of quantised rows in one launch, up to 32 tokens (see prep_small_kernel). Either x (bf16
// rows, quantised here) or q4 / s4 (rows quantised before) is given.
namespace b200moe {
int prep_small(const float* partials, int64_t stride_t, int64_t stride_s, int splits, const float* bias, int64_t tokens,
               int num_experts, int mode, float scale, int bm, float* out_w, int32_t* out_ids, int32_t* sorted_ids,
               float* sorted_w, int32_t* block_expert, int32_t* num_valid, const void* x_bf16, const uint8_t* q4,
               const uint8_t* s4, int64_t max_rows, uint8_t* xq_sorted, uint8_t* sfx, int32_t* done, int n_done,
               void* stream) {
  if (!partials || !out_w || !out_ids || !sorted_ids || !sorted_w || !block_expert || !num_valid || !xq_sorted || !sfx)
    return B200MOE_E_ARG;
  if ((x_bf16 == nullptr) == (q4 == nullptr) || (q4 != nullptr && s4 == nullptr)) return B200MOE_E_ARG;
  if (tokens < 1 || tokens > kFusedRouteTokens || num_experts < 4 || num_experts > kMaxE || splits < 1 || bm != 16 ||
      max_rows > kPrepMaxRows)
    return B200MOE_E_ARG;
  if (mode != B200MOE_ROUTE_SIGMOID_BIAS && mode != B200MOE_ROUTE_SOFTMAX) return B200MOE_E_ARG;
  const int shift = shift_of(bm);
  const unsigned grid = static_cast<unsigned>(max_rows / 4 < 1 ? 1 : (max_rows / 4 > 148 ? 148 : max_rows / 4));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint4* x = static_cast<const uint4*>(x_bf16);
#define B200MOE_PREP(M, G)                                                                                              \
  B200MOE_LAUNCH((prep_small_kernel<M, G>), grid, kChunk, 0, s, partials, stride_t, stride_s, splits, bias,             \
                 static_cast<int>(tokens), num_experts, scale, shift, out_w, out_ids, sorted_ids, sorted_w, block_expert, \
                 num_valid, x, q4, s4, xq_sorted, sfx, done, n_done)
  if (mode == B200MOE_ROUTE_SIGMOID_BIAS) {
    if (q4) B200MOE_PREP(B200MOE_ROUTE_SIGMOID_BIAS, true);
    else B200MOE_PREP(B200MOE_ROUTE_SIGMOID_BIAS, false);
  } else {
    if (q4) B200MOE_PREP(B200MOE_ROUTE_SOFTMAX, true);
    else B200MOE_PREP(B200MOE_ROUTE_SOFTMAX, false);
  }
#undef B200MOE_PREP
  return 0;
}
}  // namespace b200moe

// ------------------------------------------------------------------------------------------------ allocation-free sort
// Some hosts of this library may not allocate device memory around a call: a serving engine that hands every plugin a
// fixed memory budget at start-up and forbids cudaMalloc afterwards (it synchronises the whole device and would stall
// the other streams), or code that runs while a stream is being captured, where an allocation is an error. For them the
// chunk-count scratch of the routing sort lives in the library image itself. Every GPU that loads the library carries
// these 16 KB until the process exits.
namespace b200moe {
constexpr int kStaticSortTokens = B200MOE_STATIC_SORT_MAX_TOKENS;
constexpr int kStaticSortChunks = kStaticSortTokens * kTopK / kChunk;
static __device__ __align__(256) int32_t g_sort_scratch[kStaticSortChunks * kMaxE];

// The device address of g_sort_scratch on the CURRENT device. In host code the symbol's name is only a handle, so the
// address is looked up once per device (with that device current) and remembered.
static int static_sort_scratch(int32_t** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int32_t* ptrs[kMaxDevices] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return B200MOE_E_ARG;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_sort_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    ptrs[dev] = static_cast<int32_t*>(p);
  }
  *out = ptrs[dev];
  return 0;
}
}  // namespace b200moe

extern "C" int b200moe_permute_static(const int32_t* ids, const float* w, int64_t tokens, int num_experts, int bm,
                                      int32_t* sorted_ids, float* sorted_w, int32_t* block_expert, int32_t* num_valid,
                                      void* stream) {
  using namespace b200moe;
  if (tokens > kStaticSortTokens) return B200MOE_E_TOO_LARGE;
  int32_t* scratch = nullptr;
  const int r = static_sort_scratch(&scratch);
  if (r) return r;
  // The count pass writes every entry the placement pass reads, so nothing in the array has to start at zero.
  return b200moe_permute(ids, w, tokens, num_experts, bm, sorted_ids, sorted_w, block_expert, num_valid, scratch, stream);
}
