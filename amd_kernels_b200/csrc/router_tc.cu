// Router GEMM on the tensor cores for prefill sizes: bf16 activations x the fp32 gate carried as three bf16 terms
// (hi = RN(w), mid = RN(w - hi), lo = RN(w - hi - mid), the split of the reference's router,
// amd_kernels/moe/mxfp4_h6144_i768_e128_top4/router_gemm.py:32-44), tcgen05.mma kind::f16 with fp32 accumulators in tensor
// memory. Output: the split-K partials fp32 [S][T][E] the top-4 kernel adds in split order, the layout b200moe_router_gemm
// writes on the CUDA cores.
//
// A unit is (block of 128 tokens, K split): the token block is the 128-row M operand (TMA, 128-byte swizzle; rows past T
// are filled with zeros by the copy engine), the 128 experts are N, and each 64-element K step issues four K = 16 MMAs per
// gate term (hi, mid, lo in turn) into one accumulator, so a partial is the fp32 sum of exact bf16 products.
//
//   warp 0    producer: one thread, four tile loads per stage (tokens, gate hi / mid / lo)
//   warp 1    allocates tensor memory; one thread issues the MMAs
//   warps 2-5 epilogue: thread = token row (TMEM lane), 128 logits -> partials[s][t][0..E)
#include "tc_host.cuh"
#include "tc_ptx.cuh"

namespace b200moe {

struct RouterCfg {
  static constexpr int kStages = 3;
  static constexpr int kTileBytes = 128 * 128;            // 128 rows x 64 bf16
  static constexpr int kStageBytes = 4 * kTileBytes;      // tokens, gate hi, mid, lo
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr int kThreads = 192;
  static constexpr int kTmemCols = 256;                   // two accumulators of 128 columns
  static constexpr int kKSteps = kH / 64;                 // 96 K steps of 64 elements over the hidden size
};

__device__ __forceinline__ void tc_mma_bf16_lo(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .b64 da, db;\n.reg .pred p;\nmov.b64 da, {%1, %5};\nmov.b64 db, {%2, %5};\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n}\n" ::"r"(d),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "n"(kOperandDescHi)
      : "memory");
}

// gate fp32 [E][6144] -> three bf16 terms [3][128][6144]; rows from E on are zero
__global__ void __launch_bounds__(256) split_gate_kernel(const float* __restrict__ gate, int num_experts,
                                                         __nv_bfloat16* __restrict__ out) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<int64_t>(kMaxE) * kH) return;
  const int e = static_cast<int>(i / kH);
  float w = e < num_experts ? gate[i] : 0.0f;
#pragma unroll
  for (int p = 0; p < 3; ++p) {
    const __nv_bfloat16 t = __float2bfloat16_rn(w);
    out[static_cast<int64_t>(p) * kMaxE * kH + i] = t;
    w -= __bfloat162float(t);  // exact: the remainder of a round-to-nearest fits fp32
  }
}

__global__ void __launch_bounds__(RouterCfg::kThreads, 1)
    router_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_g,
                     float* __restrict__ partials, int64_t tokens, int num_experts, int splits, int32_t* status) {
  using C = RouterCfg;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[C::kStages];
  __shared__ __align__(8) uint64_t bar_empty[C::kStages];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ __align__(8) uint64_t bar_drain;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile int* abort_v = &abort_flag;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_tfull[a]), 1);
      mbar_init(smem_u32(&bar_tempty[a]), 128);
    }
    mbar_init(smem_u32(&bar_drain), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(static_cast<uint32_t>(C::kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  pdl_wait();

  const int blocks = static_cast<int>((tokens + 127) / 128);
  const int total_units = blocks * splits;
  const int steps = C::kKSteps / splits;  // K steps of one split

  if (warp == 0) {
    if (lane == 0) {  // ------------------------------------------------ producer
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        const int tb = u / splits, sp = u % splits;
        for (int i = 0; i < steps; ++i, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_v, status)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[s]), base = tiles + s * C::kStageBytes;
          const int kbyte = (sp * steps + i) * 128;
          mbar_arrive_expect_tx(full, C::kStageBytes);
          tma_load_2d(base, &map_x, kbyte, tb * 128, full);
          tma_load_2d(base + C::kTileBytes, &map_g, kbyte, 0, full);
          tma_load_2d(base + 2 * C::kTileBytes, &map_g, kbyte, kMaxE, full);
          tma_load_2d(base + 3 * C::kTileBytes, &map_g, kbyte, 2 * kMaxE, full);
        }
      }
      if (!ok) drain_copies(bar_full, it, C::kStages);
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ------------------------------------------------ MMA issue
      // bf16 x bf16 -> fp32, both operands K-major, M = 128 token rows, N = 128 experts
      constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(128 >> 3) << 17) |
                                  (static_cast<uint32_t>(128 >> 4) << 24);
      uint32_t it = 0, ui = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++ui) {
        const uint32_t acc = ui & 1u, aph = (ui >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tempty[acc]), aph ^ 1u, abort_v, status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * 128u;
        for (int i = 0; i < steps; ++i, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_v, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t x_lo = (tiles + s * C::kStageBytes) >> 4;
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {  // 16 K-elements = 32 bytes (descriptor + 2) per MMA
#pragma unroll
            for (int p = 1; p <= 3; ++p)
              tc_mma_bf16_lo(d_tmem, x_lo + 2 * k4, x_lo + p * (C::kTileBytes >> 4) + 2 * k4, kIdesc,
                             static_cast<uint32_t>(i != 0 || k4 != 0 || p != 1));
          }
          tc_commit(smem_u32(&bar_empty[s]));
        }
        if (ok) tc_commit(smem_u32(&bar_tfull[acc]));
      }
      if (*abort_v) drain_tcgen05(smem_u32(&bar_drain));
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    const int tr = q * 32 + lane;
    uint32_t ui = 0;
    for (int u = blockIdx.x; u < total_units; u += gridDim.x, ++ui) {
      const int tb = u / splits, sp = u % splits;
      const uint32_t acc = ui & 1u, aph = (ui >> 1) & 1u;
      if (!epilogue_all(mbar_wait(smem_u32(&bar_tfull[acc]), aph, abort_v, status), 1u)) break;
      tc_fence_after();
      const int64_t t = static_cast<int64_t>(tb) * 128 + tr;
      float* dst = partials + (static_cast<int64_t>(sp) * tokens + t) * num_experts;
      const uint32_t t_acc = tmem_base + acc * 128u + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tc_ld32(t_acc + 32 * c, v);
        if (c == 3) {  // accumulator read: hand it back to the MMA thread
          tc_fence_before();
          mbar_arrive(smem_u32(&bar_tempty[acc]));
        }
        if (t < tokens) {
          if (num_experts == kMaxE) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              *reinterpret_cast<uint4*>(dst + 32 * c + 4 * k) = make_uint4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
          } else {
#pragma unroll
            for (int k = 0; k < 32; ++k)
              if (32 * c + k < num_experts) dst[32 * c + k] = __uint_as_float(v[k]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(C::kTmemCols))
                 : "memory");
  }
}

int set_wait_limit_router(unsigned long long ns) { return set_wait_limit_here(ns); }

}  // namespace b200moe

extern "C" int b200moe_router_split_gate(const float* gate, int num_experts, void* split_bf16, void* stream) {
  using namespace b200moe;
  if (!gate || !split_bf16 || num_experts < 1 || num_experts > kMaxE) return B200MOE_E_ARG;
  if (misaligned(split_bf16, 16)) return B200MOE_E_ALIGN;
  const int64_t n = static_cast<int64_t>(kMaxE) * kH;
  B200MOE_LAUNCH_PLAIN(split_gate_kernel, static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream),
                       gate, num_experts, static_cast<__nv_bfloat16*>(split_bf16));
  return 0;
}

extern "C" int b200moe_router_gemm_tc(const void* x_bf16, const void* gate_split_bf16, int64_t tokens, int num_experts,
                                      int splits, float* partials, int32_t* status, void* stream) {
  using namespace b200moe;
  using C = RouterCfg;
  if (!x_bf16 || !gate_split_bf16 || !partials || !status || tokens < 0 || num_experts < 1 || num_experts > kMaxE)
    return B200MOE_E_ARG;
  if (splits < 1 || C::kKSteps % splits) return B200MOE_E_ARG;
  if (misaligned(x_bf16, 16) || misaligned(gate_split_bf16, 16) || misaligned(partials, 16)) return B200MOE_E_ALIGN;
  if (tokens == 0) return 0;
  CUtensorMap mx, mg;
  int r = make_map(&mx, x_bf16, kH * 2, static_cast<uint64_t>(tokens), 128);
  if (r) return r;
  if ((r = make_map(&mg, gate_split_bf16, kH * 2, 3 * kMaxE, 128))) return r;
  static PerDeviceOnce once;
  const int rc = once.run([] {
    return static_cast<int>(cudaFuncSetAttribute(router_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
  });
  if (rc) return rc;
  const int64_t units = (tokens + 127) / 128 * splits;
  const int grid = static_cast<int>(units < sm_count() ? units : sm_count());
  B200MOE_LAUNCH(router_tc_kernel, grid, C::kThreads, C::kSmemBytes, static_cast<cudaStream_t>(stream), mx, mg, partials,
                 tokens, num_experts, splits, status);
  return 0;
}
