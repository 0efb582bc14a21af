// Load-time byte permutations of the checkpoint tensors into the tile streams the tcgen05 kernels read.
//
// A weight tile = 128 rows x 256 K-elements (128 bytes per row) + its 1024 bytes of block scales, stored as ONE
// contiguous 17408-byte record, already in the shared-memory image the MMA descriptor expects:
//   bytes [0, 16384): row r, 16-byte chunk c at r*128 + ((c ^ (r & 7)) * 16)   (the 128-byte swizzle)
//   bytes [16384, 17408): two scale atoms (K elements 0..127 and 128..255 of the tile)
// so a stage of the GEMM pipeline is filled by a single bulk copy of consecutive HBM bytes.
#include "common.cuh"

namespace b200moe {

// checkpoint row of tile row r in W13 tile t: gate rows 0..767, up rows 768..1535
__device__ __forceinline__ int w13_source_row(int t, int r) {
  const int g = r >> 5;
  const int i = 64 * t + 32 * (g >> 1) + (r & 31);
  return (g & 1) ? kI + i : i;
}

// One CTA per (tile row, m-tile, expert) of at least K_BYTES / 16 threads; thread j moves 16-byte chunk j of the row and
// scale byte j.
template <int K_BYTES, int TILES_M, bool IS_W13>
__global__ void preshuffle_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                  uint8_t* __restrict__ out) {
  constexpr int kChunks = K_BYTES / 16, kScaleCols = K_BYTES / 16, kTilesK = K_BYTES / 128;
  constexpr int kRowsPerExpert = TILES_M * 128;
  const int e = blockIdx.z, t = blockIdx.y, r = blockIdx.x, j = threadIdx.x;
  const int src_row = IS_W13 ? w13_source_row(t, r) : t * 128 + r;
  const int64_t src = static_cast<int64_t>(e) * kRowsPerExpert + src_row;
  uint8_t* tile0 = out + (static_cast<int64_t>(e) * TILES_M + t) * kTilesK * kTileRecordBytes;
  if (j < kChunks) {
    const int kt = j >> 3, c = j & 7;
    const uint4 v = reinterpret_cast<const uint4*>(codes + src * K_BYTES)[j];
    *reinterpret_cast<uint4*>(tile0 + static_cast<int64_t>(kt) * kTileRecordBytes + r * 128 + ((c ^ (r & 7)) << 4)) = v;
  }
  if (j < kScaleCols) {
    // scale column j: K-tile j/8, atom (j%8)/4, byte j%4
    const int kt = j >> 3, a = (j >> 2) & 1;
    tile0[static_cast<int64_t>(kt) * kTileRecordBytes + 128 * 128 + a * kAtomBytes + atom_offset(r, j & 3)] =
        scales[src * kScaleCols + j];
  }
}

}  // namespace b200moe

extern "C" int b200moe_preshuffle_w13(const uint8_t* w13, const uint8_t* w13_scale, int num_experts, uint8_t* w13t,
                                      void* stream) {
  using namespace b200moe;
  if (!w13 || !w13_scale || !w13t || num_experts < 1 || num_experts > kMaxE) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(w13) & 15) || (reinterpret_cast<uintptr_t>(w13t) & 15)) return B200MOE_E_ALIGN;
  B200MOE_LAUNCH_PLAIN((preshuffle_kernel<kH / 2, kW13Tiles, true>), dim3(128, kW13Tiles, num_experts), (kH / 2 / 16 + 31) / 32 * 32, 0, static_cast<cudaStream_t>(stream), w13, w13_scale, w13t);
  return 0;
}

extern "C" int b200moe_preshuffle_w2(const uint8_t* w2, const uint8_t* w2_scale, int num_experts, uint8_t* w2t,
                                     void* stream) {
  using namespace b200moe;
  if (!w2 || !w2_scale || !w2t || num_experts < 1 || num_experts > kMaxE) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(w2) & 15) || (reinterpret_cast<uintptr_t>(w2t) & 15)) return B200MOE_E_ALIGN;
  B200MOE_LAUNCH_PLAIN((preshuffle_kernel<kI / 2, kW2Tiles, false>), dim3(128, kW2Tiles, num_experts), (kI / 2 / 16 + 31) / 32 * 32, 0, static_cast<cudaStream_t>(stream), w2, w2_scale, w2t);
  return 0;
}
