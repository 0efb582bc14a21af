// bf16 -> MXFP4 activation quantisation (row-major) and the gather of quantised rows into sorted order.
#include "common.cuh"

namespace b200moe {

// One thread = 8 consecutive bf16 (16 bytes in, 4 bytes out); 4 neighbouring threads share one 32-element block.
__global__ void __launch_bounds__(256) quant_mxfp4_kernel(const uint4* __restrict__ x, int64_t n_vec, int k,
                                                          uint32_t* __restrict__ codes, uint8_t* __restrict__ scales) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool live = i < n_vec;  // n_vec is a multiple of 32 per row, so a 4-thread group is live or dead together
  uint4 raw = make_uint4(0, 0, 0, 0);
  if (live) raw = x[i];
  float v[8];
  const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(r[j] << 16);
    v[2 * j + 1] = __uint_as_float(r[j] & 0xffff0000u);
  }
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const int e = quark_even_e8m0(amax);
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) packed |= e2m1_code(v[j], e) << (4 * j);
  if (live) {
    codes[i] = packed;
    if ((threadIdx.x & 3) == 0) scales[i >> 2] = static_cast<uint8_t>(e);
  }
  (void)k;
}

// Row-major quantisation at prefill sizes: one 256-thread CTA per token row, its three 16-byte loads per thread in flight
// at once; codes [T][3072] and scales [T][192], the bits of quant_mxfp4_kernel. Used ahead of the gather so that a token is
// read and quantised once, not once per routed slot.
__global__ void __launch_bounds__(256) quant_rows_kernel(const uint4* __restrict__ x, uint8_t* __restrict__ codes,
                                                         uint8_t* __restrict__ scales) {
  pdl_enter(x);
  constexpr int kIters = kH / 8 / 256;  // 3
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x;
  const uint4* src = x + row * (kH / 8);
  uint32_t* dst = reinterpret_cast<uint32_t*>(codes + row * (kH / 2));
  uint8_t* sdst = scales + row * (kH / 32);
  uint4 raw[kIters];
#pragma unroll
  for (int it = 0; it < kIters; ++it) raw[it] = __ldcs(src + it * 256 + threadIdx.x);
#pragma unroll
  for (int it = 0; it < kIters; ++it) {
    const int idx = it * 256 + threadIdx.x;
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
    // 4 lanes share a 32-element block; lanes 0 and 16 gather four neighbouring blocks' bytes into one 4-byte store
    uint32_t sc = static_cast<uint32_t>(e);
    sc |= __shfl_down_sync(0xffffffffu, sc, 4) << 8;
    sc |= __shfl_down_sync(0xffffffffu, sc, 8) << 16;
    if ((lane & 15) == 0) *reinterpret_cast<uint32_t*>(sdst + (idx >> 4) * 4) = sc;
  }
}

// One warp per sorted row: copies the token's 3072 code bytes and scatters its 192 scale bytes into the block's atoms.
// Also zeroes `done` (may be null), the per-block completion counts of a following one-launch GEMM1+GEMM2.
__global__ void __launch_bounds__(256) dispatch_rows_kernel(const uint8_t* __restrict__ codes,
                                                            const uint8_t* __restrict__ scales,
                                                            const int32_t* __restrict__ sorted_ids,
                                                            const int32_t* __restrict__ num_valid, int64_t tokens,
                                                            int bm, int by_pair, uint8_t* __restrict__ xq_sorted,
                                                            uint8_t* __restrict__ sfx, int32_t* __restrict__ done,
                                                            int n_done) {
  pdl_enter(codes, scales, sorted_ids, num_valid);
  {
    const int64_t z = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (done != nullptr && z < n_done) done[z] = 0;
  }
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= __ldcg(num_valid)) return;
  const int sid = __ldcg(sorted_ids + row);
  const bool pad = (sid & 0x00ffffff) >= tokens;
  // source row: the token, or (by_pair) the pair 4*token+slot when every (token, slot) carries its own quantised row
  const int64_t token = by_pair ? static_cast<int64_t>(sid & 0x00ffffff) * kTopK + (sid >> 24) : (sid & 0x00ffffff);
  uint4* dst = reinterpret_cast<uint4*>(xq_sorted + row * (kH / 2));
  const uint4* src = reinterpret_cast<const uint4*>(codes + token * (kH / 2));
  uint4 v[(kH / 2) / 16 / 32];
#pragma unroll
  for (int j = 0; j < (kH / 2) / 16 / 32; ++j) v[j] = pad ? make_uint4(0, 0, 0, 0) : __ldcg(src + j * 32 + lane);
#pragma unroll
  for (int j = 0; j < (kH / 2) / 16 / 32; ++j) dst[j * 32 + lane] = v[j];
  const int64_t block = row / bm;
  const int r = static_cast<int>(row % bm);
  const uint32_t* ssrc = reinterpret_cast<const uint32_t*>(scales + token * (kH / 32));
  uint8_t* sdst = sfx + block * (kH / 128) * kAtomBytes + atom_offset(r, 0);
  for (int a = lane; a < kH / 128; a += 32)  // a padding row: zero codes, the scale byte of an all-zero block
    *reinterpret_cast<uint32_t*>(sdst + a * kAtomBytes) = pad ? 0x01010101u : __ldcg(ssrc + a);
}

// Quantisation fused with the gather: one 256-thread CTA per sorted row reads the token's bf16 row (three 16-byte loads
// per thread, all in flight at once), quantises it and writes the codes in sorted order and the scales into the block's
// atoms (a token is quantised once per slot; the repeated reads hit L2).
__global__ void __launch_bounds__(256) quant_dispatch_kernel(const uint4* __restrict__ x,
                                                             const int32_t* __restrict__ sorted_ids,
                                                             const int32_t* __restrict__ num_valid, int64_t tokens,
                                                             int bm_shift, uint8_t* __restrict__ xq_sorted,
                                                             uint8_t* __restrict__ sfx, int32_t* __restrict__ done,
                                                             int n_done) {
  pdl_enter(x, sorted_ids, num_valid);
  {  // the per-block completion counts of the one-launch GEMM1+GEMM2 start every call at zero
    const int64_t z = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (done != nullptr && z < n_done) done[z] = 0;
  }
  const int64_t row = blockIdx.x;
  if (row >= __ldcg(num_valid)) return;
  const int64_t token = __ldcg(sorted_ids + row) & 0x00ffffff;
  uint32_t* dst = reinterpret_cast<uint32_t*>(xq_sorted + row * (kH / 2));
  const int r = static_cast<int>(row & ((1 << bm_shift) - 1));
  uint8_t* sdst = sfx + (row >> bm_shift) * (kH / 128) * kAtomBytes + atom_offset(r, 0);
  quant_row_to_atoms(token >= tokens ? nullptr : x + token * (kH / 8), dst, sdst, threadIdx.x);
}

// Expert-parallel dispatch fused with the quantisation: one CTA per send row quantises the pair's token row and stores
// codes (3072 contiguous bytes), row-major scales (192 bytes) and four meta words {expert id on the destination, routing
// weight bits, source pair, source rank} (column arrays [4][capacity]) straight into the destination rank's receive buffers (peer mappings over
// NVLink, or local memory for rows that stay). Plain stores, no waits; the caller orders the ranks afterwards.
struct PushArgs {
  uint8_t* codes[8];
  uint8_t* scales[8];
  int32_t* meta[8];
  const int64_t* dst_base;   // device [world]: first row of this rank's segment in each destination's buffers
  const int32_t* seg_start;  // device [world]: first send row that goes to each destination
  int32_t world, rank, experts_per_rank, interleaved;
  int64_t capacity;      // rows every receive buffer holds
};

__global__ void __launch_bounds__(256) quant_push_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ ids,
                                                         const int32_t* __restrict__ send_ids,
                                                         const float* __restrict__ send_w,
                                                         const int32_t* __restrict__ send_rank, int64_t tokens,
                                                         PushArgs a, int32_t* status) {
  // One WARP per send row, eight rows per CTA: a row's chain of dependent loads (send entry -> destination -> offsets ->
  // the token's row) is short work for 256 threads, and with one CTA per row the kernel was bound by that latency (measured
  // 105-134 us for 16384 rows at 4 ranks against ~52 us of NVLink time). A lane owns the 16-byte chunks lane, lane + 32,
  // ... of the row (8 values each); four neighbouring lanes share a 32-value block.
  constexpr int kChunks = kH / 8 / 32;  // 24 chunks per lane
  constexpr int kBatch = 8;
  __shared__ __align__(16) uint32_t s_scales[8][kH / 128];  // a row's 192 scale bytes, per warp
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  if (i >= tokens * kTopK) return;
  const int sid = send_ids[i];
  const int64_t token = sid & 0x00ffffff;
  const int slot = (sid >> 24) & 3, d = send_rank[i];
  if (token >= tokens || d < 0 || d >= a.world) return;
  const int64_t row = __ldg(a.dst_base + d) + (i - __ldg(a.seg_start + d));
  if (row < 0 || row >= a.capacity) {  // never store outside a receive buffer
    if (lane == 0) atomicExch(status, B200MOE_DEV_BAD_INDEX);
    return;
  }
  const uint4* src = x + token * (kH / 8);
  uint32_t* dst = reinterpret_cast<uint32_t*>(a.codes[d] + row * (kH / 2));
#pragma unroll 1
  for (int b0 = 0; b0 < kChunks; b0 += kBatch) {
    uint4 raw[kBatch];
#pragma unroll
    for (int it = 0; it < kBatch; ++it) raw[it] = src[(b0 + it) * 32 + lane];
#pragma unroll
    for (int it = 0; it < kBatch; ++it) {
      const int idx = (b0 + it) * 32 + lane;
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
      const float inv = __uint_as_float(static_cast<uint32_t>(254 - e) << 23);
      uint32_t packed = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) packed |= cvt_e2m1x2(v[2 * j] * inv, v[2 * j + 1] * inv) << (8 * j);
      dst[idx] = packed;  // the warp writes 128 contiguous bytes: whole packets when the destination is a peer over NVLink
      uint32_t sc = static_cast<uint32_t>(e);
      sc |= __shfl_down_sync(0xffffffffu, sc, 4) << 8;
      sc |= __shfl_down_sync(0xffffffffu, sc, 8) << 16;
      if ((lane & 15) == 0) s_scales[warp][idx >> 4] = sc;  // scale bytes 4*(idx/16) .. +3 of the row
    }
  }
  __syncwarp();
  if (lane < kH / 512)
    reinterpret_cast<uint4*>(a.scales[d] + row * (kH / 32))[lane] = reinterpret_cast<const uint4*>(s_scales[warp])[lane];
  if (lane == 0) {
    const int e = ids[token * kTopK + slot];
    const int local = a.interleaved ? e / a.world : e % a.experts_per_rank;
    // four column arrays [4][capacity]: the receiver hands columns straight to its sort and to GEMM2's row tables
    int32_t* m = a.meta[d] + row;
    m[0] = local;
    m[a.capacity] = __float_as_int(send_w[i]);
    m[2 * a.capacity] = static_cast<int>(token * kTopK + slot);
    m[3 * a.capacity] = a.rank;
  }
}

}  // namespace b200moe

namespace b200moe {
int quant_rows(const void* x_bf16, int64_t tokens, uint8_t* codes, uint8_t* scales, void* stream);
}

extern "C" int b200moe_quant_push(const void* x_bf16, const int32_t* ids, const int32_t* send_ids, const float* send_w,
                                  const int32_t* send_rank, int64_t tokens, int world, int rank, int experts_per_rank,
                                  int interleaved, void* const* peer_codes, void* const* peer_scales,
                                  void* const* peer_meta, const int64_t* dst_base, const int32_t* seg_start,
                                  int64_t capacity, int32_t* status, void* stream) {
  using namespace b200moe;
  if (!x_bf16 || !ids || !send_ids || !send_w || !send_rank || !peer_codes || !peer_scales || !peer_meta || !dst_base ||
      !seg_start || !status)
    return B200MOE_E_ARG;
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS || world < 1 || world > 8 || rank < 0 || rank >= world ||
      experts_per_rank < 1 || capacity < 1)
    return B200MOE_E_ARG;
  PushArgs a{};
  for (int r = 0; r < 8; ++r) {
    const int k = r < world ? r : 0;
    a.codes[r] = static_cast<uint8_t*>(peer_codes[k]);
    a.scales[r] = static_cast<uint8_t*>(peer_scales[k]);
    a.meta[r] = static_cast<int32_t*>(peer_meta[k]);
    if (!a.codes[r] || !a.scales[r] || !a.meta[r]) return B200MOE_E_ARG;
    if ((reinterpret_cast<uintptr_t>(a.codes[r]) | reinterpret_cast<uintptr_t>(a.scales[r]) |
         reinterpret_cast<uintptr_t>(a.meta[r])) & 15)
      return B200MOE_E_ALIGN;
  }
  a.dst_base = dst_base;
  a.seg_start = seg_start;
  a.world = world;
  a.rank = rank;
  a.experts_per_rank = experts_per_rank;
  a.interleaved = interleaved;
  a.capacity = capacity;
  if (reinterpret_cast<uintptr_t>(x_bf16) & 15) return B200MOE_E_ALIGN;
  B200MOE_LAUNCH_PLAIN(quant_push_kernel, static_cast<unsigned>((tokens * kTopK + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream),
                       static_cast<const uint4*>(x_bf16), ids, send_ids, send_w, send_rank, tokens, a, status);
  return 0;
}

extern "C" int b200moe_quant_mxfp4(const void* x_bf16, int64_t tokens, int k, uint8_t* codes, uint8_t* scales,
                                   void* stream) {
  using namespace b200moe;
  if (!x_bf16 || !codes || !scales || tokens < 0 || k <= 0 || (k % 256) != 0) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(codes) & 3)) return B200MOE_E_ALIGN;
  if (tokens == 0) return 0;
  if (k == kH && tokens >= 64) return b200moe::quant_rows(x_bf16, tokens, codes, scales, stream);
  const int64_t n_vec = tokens * (k / 8);
  const unsigned grid = static_cast<unsigned>((n_vec + 255) / 256);
  B200MOE_LAUNCH_PLAIN(quant_mxfp4_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream), static_cast<const uint4*>(x_bf16), n_vec, k, reinterpret_cast<uint32_t*>(codes), scales);
  return 0;
}

namespace b200moe {
int quant_rows(const void* x_bf16, int64_t tokens, uint8_t* codes, uint8_t* scales, void* stream) {
  if (!x_bf16 || !codes || !scales || tokens < 0) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(codes) & 3) ||
      (reinterpret_cast<uintptr_t>(scales) & 3))
    return B200MOE_E_ALIGN;
  if (tokens == 0) return 0;
  B200MOE_LAUNCH(quant_rows_kernel, static_cast<unsigned>(tokens), 256, 0, static_cast<cudaStream_t>(stream),
                 static_cast<const uint4*>(x_bf16), codes, scales);
  return 0;
}

int dispatch_rows_done(const uint8_t* codes, const uint8_t* scales, const int32_t* sorted_ids, const int32_t* num_valid,
                       int64_t tokens, int bm, int by_pair, int64_t max_rows, uint8_t* xq_sorted, uint8_t* sfx,
                       int32_t* done, void* stream) {
  if (!codes || !scales || !sorted_ids || !num_valid || !xq_sorted || !sfx || tokens < 0 || max_rows < 0)
    return B200MOE_E_ARG;
  if (bm != 16 && bm != 32 && bm != 64 && bm != 128) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(xq_sorted) & 15) ||
      (reinterpret_cast<uintptr_t>(scales) & 3) || (reinterpret_cast<uintptr_t>(sfx) & 15))
    return B200MOE_E_ALIGN;
  if (max_rows == 0) return 0;
  const unsigned grid = static_cast<unsigned>((max_rows + 7) / 8);
  B200MOE_LAUNCH(dispatch_rows_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream), codes, scales, sorted_ids,
                 num_valid, tokens, bm, by_pair, xq_sorted, sfx, done, static_cast<int>(max_rows / bm));
  return 0;
}
}  // namespace b200moe

extern "C" int b200moe_dispatch_rows(const uint8_t* codes, const uint8_t* scales, const int32_t* sorted_ids,
                                     const int32_t* num_valid, int64_t tokens, int bm, int by_pair, int64_t max_rows,
                                     uint8_t* xq_sorted, uint8_t* sfx, void* stream) {
  return b200moe::dispatch_rows_done(codes, scales, sorted_ids, num_valid, tokens, bm, by_pair, max_rows, xq_sorted, sfx,
                                     nullptr, stream);
}

extern "C" int b200moe_quant_dispatch(const void* x_bf16, const int32_t* sorted_ids, const int32_t* num_valid,
                                      int64_t tokens, int bm, int64_t max_rows, uint8_t* xq_sorted, uint8_t* sfx,
                                      int32_t* done, void* stream) {
  using namespace b200moe;
  if (!x_bf16 || !sorted_ids || !num_valid || !xq_sorted || !sfx || tokens < 0 || max_rows < 0) return B200MOE_E_ARG;
  const int shift = bm == 16 ? 4 : bm == 32 ? 5 : bm == 64 ? 6 : bm == 128 ? 7 : -1;
  if (shift < 0) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(xq_sorted) & 15) ||
      (reinterpret_cast<uintptr_t>(sfx) & 15))
    return B200MOE_E_ALIGN;
  if (max_rows == 0) return 0;
  const unsigned grid = static_cast<unsigned>(max_rows);
  B200MOE_LAUNCH(quant_dispatch_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream), static_cast<const uint4*>(x_bf16), sorted_ids, num_valid, tokens, shift, xq_sorted, sfx, done, static_cast<int>(max_rows / bm));
  return 0;
}
