// The compact prepared input: the routed experts' FP4 codes are not sent; the receiver rebuilds them bit for bit from the
// shared expert's FP8 codes of the same row, both scale rows and one correction bit per value.
// candidate(v) = the FP4 code of |e4m3(v)| / 2^(s4 - s8) with the thresholds .25 .75 1.25 1.75 2.5 3.5 5 (ties to the even
// code), sign from the FP8 byte; mask bit = (candidate != direct code). One thread = 8 values = one mask byte.
#include "common.cuh"

namespace b200moe {

__device__ __forceinline__ float e4m3_magnitude(uint32_t byte) {
  const uint32_t e = (byte >> 3) & 15u, m = byte & 7u;
  // normal: (1 + m/8) * 2^(e-7); subnormal: m * 2^-9
  return e ? __uint_as_float(((e + 120u) << 23) | (m << 20)) : static_cast<float>(m) * 0.001953125f;
}

// magnitude in FP4 units and the candidate code (sign in bit 3)
__device__ __forceinline__ uint32_t candidate_code(uint32_t q8, float inv_ratio, float& magnitude) {
  magnitude = e4m3_magnitude(q8) * inv_ratio;  // a power of two: exact
  const uint32_t c = (magnitude > 0.25f) + (magnitude >= 0.75f) + (magnitude > 1.25f) + (magnitude >= 1.75f) +
                     (magnitude > 2.5f) + (magnitude >= 3.5f) + (magnitude > 5.0f);
  return c | ((q8 >> 7) << 3);
}

__device__ __forceinline__ float inverse_ratio(const uint8_t* s4, const uint8_t* s8, int64_t row, int col) {
  const int d = static_cast<int>(s8[row * (kH / 32) + (col >> 5)]) - static_cast<int>(s4[row * (kH / 32) + (col >> 5)]);
  return __uint_as_float(static_cast<uint32_t>(min(max(d, -126), 127) + 127) << 23);  // 2^(s8 - s4), exact
}

__global__ void __launch_bounds__(256) sidecar_pack_kernel(const uint32_t* __restrict__ q4, const uint8_t* __restrict__ s4,
                                                           const uint2* __restrict__ q8, const uint8_t* __restrict__ s8,
                                                           int64_t n_bytes, uint8_t* __restrict__ mask) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;  // mask byte = values 8i .. 8i+7
  if (i >= n_bytes) return;
  const int64_t row = i / (kH / 8);
  const int col = static_cast<int>(i % (kH / 8)) * 8;
  const float inv = inverse_ratio(s4, s8, row, col);
  const uint32_t direct = q4[i];
  const uint2 b8 = q8[i];
  uint32_t bits = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t byte = ((j < 4 ? b8.x : b8.y) >> (8 * (j & 3))) & 255u;
    float mag;
    const uint32_t cand = candidate_code(byte, inv, mag);
    bits |= static_cast<uint32_t>(cand != ((direct >> (4 * j)) & 15u)) << j;
  }
  mask[i] = static_cast<uint8_t>(bits);
}

__global__ void __launch_bounds__(256) sidecar_unpack_kernel(const uint8_t* __restrict__ mask, const uint8_t* __restrict__ s4,
                                                             const uint2* __restrict__ q8, const uint8_t* __restrict__ s8,
                                                             int64_t n_bytes, uint32_t* __restrict__ q4) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= n_bytes) return;
  const int64_t row = i / (kH / 8);
  const int col = static_cast<int>(i % (kH / 8)) * 8;
  const float inv = inverse_ratio(s4, s8, row, col);
  const uint32_t bits = mask[i];
  const uint2 b8 = q8[i];
  uint32_t out = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t byte = ((j < 4 ? b8.x : b8.y) >> (8 * (j & 3))) & 255u;
    float mag;
    uint32_t code = candidate_code(byte, inv, mag);
    if ((bits >> j) & 1u) {
      // the other neighbour: below at the midpoints that round up (.75, 1.75, 3.5), above elsewhere
      const bool down = mag == 0.75f || mag == 1.75f || mag == 3.5f;
      code = (code & 8u) | (((code & 7u) + (down ? 7u : 1u)) & 7u);
    }
    out |= code << (4 * j);
  }
  q4[i] = out;
}

// row-major scale bytes [tokens][cols] -> the scale atoms of bm-row blocks [ceil(tokens/bm)][cols/4][512]; rows of the
// last block beyond `tokens` get the scale byte 1
__global__ void __launch_bounds__(256) scales_to_atoms_kernel(const uint8_t* __restrict__ rows, int64_t tokens, int cols,
                                                              int bm_shift, int64_t padded_rows, uint8_t* __restrict__ atoms) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;  // one 4-byte cell: (row, cols/4)
  const int cells = cols >> 2;
  if (i >= padded_rows * cells) return;
  const int64_t row = i / cells;
  const int a = static_cast<int>(i % cells);
  const uint32_t v = row < tokens ? *reinterpret_cast<const uint32_t*>(rows + row * cols + 4 * a) : 0x01010101u;
  const int r = static_cast<int>(row & ((1 << bm_shift) - 1));
  *reinterpret_cast<uint32_t*>(atoms + ((row >> bm_shift) * cells + a) * kAtomBytes + atom_offset(r, 0)) = v;
}

}  // namespace b200moe

static int sidecar_args(const void* a, const void* b, const void* c, const void* d, const void* e, int64_t tokens) {
  if (!a || !b || !c || !d || !e || tokens < 0 || tokens > B200MOE_MAX_TOKENS) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(e)) & 7)
    return B200MOE_E_ALIGN;
  return 0;
}

extern "C" int b200moe_sidecar_pack(const uint8_t* q4, const uint8_t* s4, const uint8_t* q8, const uint8_t* s8,
                                    int64_t tokens, uint8_t* mask, void* stream) {
  using namespace b200moe;
  const int r = sidecar_args(q4, s4, q8, s8, mask, tokens);
  if (r || tokens == 0) return r;
  const int64_t n = tokens * (kH / 8);
  B200MOE_LAUNCH_PLAIN(sidecar_pack_kernel, static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream),
                       reinterpret_cast<const uint32_t*>(q4), s4, reinterpret_cast<const uint2*>(q8), s8, n, mask);
  return 0;
}

extern "C" int b200moe_sidecar_unpack(const uint8_t* mask, const uint8_t* s4, const uint8_t* q8, const uint8_t* s8,
                                      int64_t tokens, uint8_t* q4, void* stream) {
  using namespace b200moe;
  const int r = sidecar_args(q4, s4, q8, s8, mask, tokens);
  if (r || tokens == 0) return r;
  const int64_t n = tokens * (kH / 8);
  B200MOE_LAUNCH_PLAIN(sidecar_unpack_kernel, static_cast<unsigned>((n + 255) / 256), 256, 0,
                       static_cast<cudaStream_t>(stream), mask, s4, reinterpret_cast<const uint2*>(q8), s8, n,
                       reinterpret_cast<uint32_t*>(q4));
  return 0;
}

extern "C" int b200moe_scales_to_atoms(const uint8_t* rows, int64_t tokens, int cols, int bm, uint8_t* atoms, void* stream) {
  using namespace b200moe;
  if (!rows || !atoms || tokens < 1 || tokens > B200MOE_MAX_TOKENS || cols < 4 || (cols & 3)) return B200MOE_E_ARG;
  const int shift = bm == 16 ? 4 : bm == 32 ? 5 : bm == 64 ? 6 : bm == 128 ? 7 : -1;
  if (shift < 0) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(rows) & 3) || (reinterpret_cast<uintptr_t>(atoms) & 15)) return B200MOE_E_ALIGN;
  const int64_t padded = (tokens + bm - 1) / bm * bm;
  const int64_t n = padded * (cols >> 2);
  B200MOE_LAUNCH_PLAIN(scales_to_atoms_kernel, static_cast<unsigned>((n + 255) / 256), 256, 0,
                       static_cast<cudaStream_t>(stream), rows, tokens, cols, shift, padded, atoms);
  return 0;
}
