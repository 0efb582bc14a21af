// Load-time byte permutations of the checkpoint tensors into the layouts the tcgen05 kernels stream.
#include "common.cuh"

namespace b200moe {

// checkpoint row of tile row r in W13 tile t: gate rows 0..767, up rows 768..1535
__device__ __forceinline__ int w13_source_row(int t, int r) {
  const int g = r >> 5;
  const int i = 64 * t + 32 * (g >> 1) + (r & 31);
  return (g & 1) ? kI + i : i;
}

// grid (12*128, E): one CTA copies one 3072-byte row and scatters its 192 scale bytes
__global__ void __launch_bounds__(192) preshuffle_w13_kernel(const uint8_t* __restrict__ w13,
                                                             const uint8_t* __restrict__ s13,
                                                             uint8_t* __restrict__ w13p, uint8_t* __restrict__ sf13p) {
  const int e = blockIdx.y, t = blockIdx.x >> 7, r = blockIdx.x & 127;
  const int64_t src = static_cast<int64_t>(e) * 2 * kI + w13_source_row(t, r);
  const int64_t dst = (static_cast<int64_t>(e) * kW13Tiles + t) * 128 + r;
  reinterpret_cast<uint4*>(w13p + dst * (kH / 2))[threadIdx.x] =
      reinterpret_cast<const uint4*>(w13 + src * (kH / 2))[threadIdx.x];
  // scale column c -> K-tile c/8, atom (c%8)/4, byte c%4
  const int c = threadIdx.x;  // 192 scale columns
  uint8_t* tile = sf13p + (static_cast<int64_t>(e) * kW13Tiles + t) * kK1Tiles * 2 * kAtomBytes;
  tile[(c >> 2) * kAtomBytes + atom_offset(r, c & 3)] = s13[src * (kH / 32) + c];
}

// grid (48*128, E), 32 threads: 24 scale columns per row
__global__ void __launch_bounds__(32) preshuffle_w2_scales_kernel(const uint8_t* __restrict__ s2,
                                                                  uint8_t* __restrict__ sf2p) {
  const int e = blockIdx.y, t = blockIdx.x >> 7, r = blockIdx.x & 127;
  const int c = threadIdx.x;
  if (c >= kI / 32) return;
  const int64_t src = static_cast<int64_t>(e) * kH + t * 128 + r;
  uint8_t* tile = sf2p + (static_cast<int64_t>(e) * kW2Tiles + t) * kK2Tiles * 2 * kAtomBytes;
  tile[(c >> 2) * kAtomBytes + atom_offset(r, c & 3)] = s2[src * (kI / 32) + c];
}

}  // namespace b200moe

extern "C" int b200moe_preshuffle_w13(const uint8_t* w13, const uint8_t* w13_scale, int num_experts, uint8_t* w13p,
                                      uint8_t* sf13p, void* stream) {
  using namespace b200moe;
  if (!w13 || !w13_scale || !w13p || !sf13p || num_experts < 1 || num_experts > kMaxE) return B200MOE_E_ARG;
  if ((reinterpret_cast<uintptr_t>(w13) & 15) || (reinterpret_cast<uintptr_t>(w13p) & 15) ||
      (reinterpret_cast<uintptr_t>(sf13p) & 15))
    return B200MOE_E_ALIGN;
  preshuffle_w13_kernel<<<dim3(kW13Tiles * 128, num_experts), 192, 0, static_cast<cudaStream_t>(stream)>>>(
      w13, w13_scale, w13p, sf13p);
  B200MOE_CHECK_LAUNCH();
  return 0;
}

extern "C" int b200moe_preshuffle_w2_scales(const uint8_t* w2_scale, int num_experts, uint8_t* sf2p, void* stream) {
  using namespace b200moe;
  if (!w2_scale || !sf2p || num_experts < 1 || num_experts > kMaxE) return B200MOE_E_ARG;
  if (reinterpret_cast<uintptr_t>(sf2p) & 15) return B200MOE_E_ALIGN;
  preshuffle_w2_scales_kernel<<<dim3(kW2Tiles * 128, num_experts), 32, 0, static_cast<cudaStream_t>(stream)>>>(
      w2_scale, sf2p);
  B200MOE_CHECK_LAUNCH();
  return 0;
}
