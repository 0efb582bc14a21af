// The MXFP8 shared expert: a dense SwiGLU MLP (6144 -> 2x768 -> 6144) on every token, E4M3 weights and activations with
// one E8M0 scale per 32 elements, on tcgen05.mma kind::mxf8f6f4 block-scaled. Same skeleton as the routed kernels:
// persistent CTAs, weight tile = the 128-row M operand, a block of bm tokens = N, TMEM accumulators, warp roles
// producer / MMA / epilogue, bounded waits. Token blocks are dense (block b = rows b*bm ..), there is no routing table.
//
// Weight records: one tile of 128 rows x 128 K-elements = 16384 bytes of E4M3 codes in the 128-byte-swizzled image,
// then one scale atom (4 scales per row), padded to 17408 bytes so the token tile behind it stays 1024-byte aligned.
#include "tc_host.cuh"
#include "tc_ptx.cuh"

namespace b200moe {

constexpr int kS1TilesK = kH / 128;  // 48 K-tiles of 128 elements in the first GEMM
constexpr int kS2TilesK = kI / 128;  // 6 in the second

// ------------------------------------------------------------------------------------------------ weight preshuffle
template <int K_BYTES, int TILES_M, bool IS_W13>
__global__ void preshuffle_shared_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                                         uint8_t* __restrict__ out) {
  constexpr int kTilesK = K_BYTES / 128, kScaleCols = K_BYTES / 32;
  const int t = blockIdx.y, r = blockIdx.x;
  int src_row = t * 128 + r;
  if (IS_W13) {  // tile rows: [gate 32 | up 32 | gate 32 | up 32] of 64 intermediate columns
    const int g = r >> 5, i = 64 * t + 32 * (g >> 1) + (r & 31);
    src_row = (g & 1) ? kI + i : i;
  }
  uint8_t* tile0 = out + static_cast<int64_t>(t) * kTilesK * kTileRecordBytes;
  for (int j = threadIdx.x; j < K_BYTES / 16; j += blockDim.x) {
    const int kt = j >> 3, c = j & 7;
    const uint4 v = reinterpret_cast<const uint4*>(codes + static_cast<int64_t>(src_row) * K_BYTES)[j];
    *reinterpret_cast<uint4*>(tile0 + static_cast<int64_t>(kt) * kTileRecordBytes + r * 128 + ((c ^ (r & 7)) << 4)) = v;
  }
  for (int j = threadIdx.x; j < kScaleCols; j += blockDim.x)
    tile0[static_cast<int64_t>(j >> 2) * kTileRecordBytes + 128 * 128 + atom_offset(r, j & 3)] =
        scales[static_cast<int64_t>(src_row) * kScaleCols + j];
}

// ------------------------------------------------------------------------------------------------ activation quant
// One 256-thread CTA per (padded) token row: bf16 -> E4M3 codes [row][6144] and the row's scales into the block's atoms.
// With `row_scales` the scale bytes go to a row-major [tokens][192] array instead of the atoms (the prepared-input payload).
__global__ void __launch_bounds__(256) shared_quant_kernel(const uint4* __restrict__ x, int64_t tokens, int bm_shift,
                                                           uint8_t* __restrict__ codes, uint8_t* __restrict__ atoms,
                                                           uint8_t* __restrict__ row_scales) {
  pdl_enter(x);
  constexpr int kIters = kH / 8 / 256;  // 3
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x;
  uint2* dst = reinterpret_cast<uint2*>(codes + row * kH);
  const int r = static_cast<int>(row & ((1 << bm_shift) - 1));
  uint8_t* sdst = atoms + (row >> bm_shift) * kS1TilesK * kAtomBytes + atom_offset(r, 0);
  if (row >= tokens) {  // padding rows of the last block
#pragma unroll
    for (int it = 0; it < kIters; ++it) {
      const int idx = it * 256 + threadIdx.x;
      dst[idx] = make_uint2(0u, 0u);
      if ((lane & 15) == 0) *reinterpret_cast<uint32_t*>(sdst + (idx >> 4) * kAtomBytes) = 0x01010101u;
    }
    return;
  }
  const uint4* src = x + row * (kH / 8);
  uint4 raw[kIters];
#pragma unroll
  for (int it = 0; it < kIters; ++it) raw[it] = src[it * 256 + threadIdx.x];
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
    const int e = mxfp8_scale(amax);
    const float inv = __uint_as_float(static_cast<uint32_t>(254 - e) << 23);  // 2^(127-e); e <= 247 here
    uint32_t w0 = cvt_e4m3x2(v[0] * inv, v[1] * inv) | (cvt_e4m3x2(v[2] * inv, v[3] * inv) << 16);
    uint32_t w1 = cvt_e4m3x2(v[4] * inv, v[5] * inv) | (cvt_e4m3x2(v[6] * inv, v[7] * inv) << 16);
    dst[idx] = make_uint2(w0, w1);
    uint32_t sc = static_cast<uint32_t>(e);
    sc |= __shfl_down_sync(0xffffffffu, sc, 4) << 8;
    sc |= __shfl_down_sync(0xffffffffu, sc, 8) << 16;
    if ((lane & 15) == 0) {
      if (row_scales != nullptr) *reinterpret_cast<uint32_t*>(row_scales + row * (kH / 32) + (idx >> 4) * 4) = sc;
      else *reinterpret_cast<uint32_t*>(sdst + (idx >> 4) * kAtomBytes) = sc;
    }
  }
}

// ------------------------------------------------------------------------------------------------ GEMM kernel
template <int MODE, int BM>
struct Cfg8 {
  static constexpr int kTilesM = MODE == 1 ? kW13Tiles : kW2Tiles;
  static constexpr int kTilesK = MODE == 1 ? kS1TilesK : kS2TilesK;
  static constexpr int kBOffset = kTileRecordBytes;
  static constexpr int kSfbOffset = kBOffset + BM * 128;
  static constexpr int kStageBytes = kSfbOffset + 1024;
  static constexpr int kTxBytes = kTileRecordBytes + BM * 128 + kAtomBytes;
  static constexpr int kStages = BM == 128 ? 5 : (BM == 64 ? 6 : 8);
  // scale columns behind the accumulators: 8 sets of (4 weight + 4 token columns) used in rotation; their copies are
  // issued by a thread of their own (warp 6), stages ahead of the MMAs
  static constexpr int kSfSets = 8;
  static constexpr int kSfaCol = 2 * BM;
  static constexpr int kColsUsed = kSfaCol + 8 * kSfSets;
  static constexpr int kTmemCols = kColsUsed <= 64 ? 64 : (kColsUsed <= 128 ? 128 : (kColsUsed <= 256 ? 256 : 512));
  static constexpr int kEpiCols = MODE == 1 ? (BM < 64 ? BM : 64) : (BM < 32 ? BM : 32);
  static constexpr int kEpiRowFloats = MODE == 1 ? 136 : 132;
  static constexpr int kEpiBytes = kEpiCols * kEpiRowFloats * 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024;
  static constexpr int kActRowBytes = MODE == 1 ? kH : kI;
};

struct SharedEpilogue {
  uint8_t* h8;           // GEMM1 out: E4M3 codes [rows][768]
  uint8_t* sfh8;         // GEMM1 out: scale atoms [rows/bm][6][512]
  __nv_bfloat16* out;    // GEMM2 out: bf16 [tokens][6144]
  int64_t tokens;
};

template <int MODE, int BM>
__global__ void __launch_bounds__(224, 1)
    shared_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const uint8_t* __restrict__ w_tiles,
                       const uint8_t* __restrict__ sf_x, int n_blocks, SharedEpilogue ep, int32_t* status) {
  using C = Cfg8<MODE, BM>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[C::kStages];
  __shared__ __align__(8) uint64_t bar_empty[C::kStages];
  __shared__ __align__(8) uint64_t bar_sf[C::kStages];
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ __align__(8) uint64_t bar_drain[2];  // used after an abort only
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
      mbar_init(smem_u32(&bar_sf[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_tfull[a]), 1);
      mbar_init(smem_u32(&bar_tempty[a]), 128);
      mbar_init(smem_u32(&bar_drain[a]), 1);
    }
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
  launder(w_tiles);
  launder(sf_x);
  const int total_units = n_blocks * C::kTilesM;

  if (warp == 0) {
    if (lane == 0) {  // ------------------------------------------------ producer
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        const int b = u / C::kTilesM, mt = u % C::kTilesM;
        const uint8_t* w_src = w_tiles + static_cast<int64_t>(mt) * C::kTilesK * kTileRecordBytes;
        const uint8_t* sfb_src = sf_x + static_cast<int64_t>(b) * C::kTilesK * kAtomBytes;
        for (int kt = 0; kt < C::kTilesK; ++kt, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_v, status)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t base = tiles + s * C::kStageBytes;
          mbar_arrive_expect_tx(full, C::kTxBytes);
          bulk_load(base, w_src + static_cast<int64_t>(kt) * kTileRecordBytes, kTileRecordBytes, full);
          tma_load_2d(base + C::kBOffset, &map_x, kt * 128, b * BM, full);
          bulk_load(base + C::kSfbOffset, sfb_src + kt * kAtomBytes, kAtomBytes, full);
        }
      }
      if (!ok) {
        drain_copies(bar_full, it, C::kStages);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ------------------------------------------------ MMA issue
      // E4M3 x E4M3 (format 0), UE8M0 scales, M = 128, N = BM; scale byte k of each row's 4-byte cell for MMA k
      constexpr uint32_t kIdesc = (static_cast<uint32_t>(BM >> 3) << 17) | (1u << 23) | (8u << 24);
      const uint32_t sf0 = smem_u32(&bar_sf[0]), empty0 = smem_u32(&bar_empty[0]);
      uint32_t slot = 0, ph = 0, sfset = 0, ui = 0;
      uint32_t lo = tiles >> 4, sf = sf0, empty = empty0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++ui) {
        const uint32_t acc = ui & 1u, aph = (ui >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tempty[acc]), aph ^ 1u, abort_v, status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BM;
        for (int kt = 0; kt < C::kTilesK; ++kt) {
          if (!mbar_wait(sf, ph, abort_v, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t t_sfa = tmem_base + C::kSfaCol + 8u * sfset, t_sfb = t_sfa + 4u;
          const uint32_t w_lo = lo, x_lo = lo + (C::kBOffset >> 4);
          // 32 elements = 32 bytes (descriptor + 2) per MMA
          tc_mma_mxf8_lo<2>(d_tmem, w_lo, x_lo, kIdesc, t_sfa, t_sfb, static_cast<uint32_t>(kt != 0));
          tc_mma_mxf8_lo<1>(d_tmem, w_lo + 2, x_lo + 2, kIdesc | (1u << 29) | (1u << 4), t_sfa, t_sfb);
          tc_mma_mxf8_lo<1>(d_tmem, w_lo + 4, x_lo + 4, kIdesc | (2u << 29) | (2u << 4), t_sfa, t_sfb);
          tc_mma_mxf8_lo<1>(d_tmem, w_lo + 6, x_lo + 6, kIdesc | (3u << 29) | (3u << 4), t_sfa, t_sfb);
          tc_commit(empty);
          sfset = (sfset + 1u) & (C::kSfSets - 1);
          if (++slot == C::kStages) {
            slot = 0; ph ^= 1u; lo = tiles >> 4; sf = sf0; empty = empty0;
          } else {
            lo += C::kStageBytes >> 4; sf += 8; empty += 8;
          }
        }
        if (ok) tc_commit(smem_u32(&bar_tfull[acc]));
      }
      if (*abort_v) drain_tcgen05(smem_u32(&bar_drain[0]));
    }
  } else if (warp == 6) {
    if (lane == 0) {  // ------------------------------------------------ scale copies: shared memory -> tensor memory
      const uint32_t full0 = smem_u32(&bar_full[0]), sf0 = smem_u32(&bar_sf[0]);
      uint32_t slot = 0, ph = 0, sfset = 0;
      uint32_t lo = tiles >> 4, full = full0, sf = sf0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        for (int kt = 0; kt < C::kTilesK; ++kt) {
          if (!mbar_wait(full, ph, abort_v, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t t_sfa = tmem_base + C::kSfaCol + 8u * sfset;
          tc_cp_scales_lo(t_sfa, lo + ((128 * 128) >> 4));
          tc_cp_scales_lo(t_sfa + 4, lo + (C::kSfbOffset >> 4));
          tc_commit(sf);
          sfset = (sfset + 1u) & (C::kSfSets - 1);
          if (++slot == C::kStages) {
            slot = 0; ph ^= 1u; lo = tiles >> 4; full = full0; sf = sf0;
          } else {
            lo += C::kStageBytes >> 4; full += 8; sf += 8;
          }
        }
      }
      if (*abort_v) drain_tcgen05(smem_u32(&bar_drain[1]));
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    float* stage_f = reinterpret_cast<float*>(smem_raw + (tiles - smem_u32(smem_raw)) + C::kStages * C::kStageBytes);
    uint32_t ui = 0;
    for (int u = blockIdx.x; u < total_units; u += gridDim.x, ++ui) {
      const int b = u / C::kTilesM, mt = u % C::kTilesM;
      const uint32_t acc = ui & 1u, aph = (ui >> 1) & 1u;
      const int64_t row0 = static_cast<int64_t>(b) * BM;
      if (!epilogue_all(mbar_wait(smem_u32(&bar_tfull[acc]), aph, abort_v, status), 1u)) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + acc * BM + (static_cast<uint32_t>(q * 32) << 16);
      float* mine = MODE == 1 ? stage_f + (q >> 1) * 68 + (q & 1) * 32 + lane : stage_f + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BM; c0 += C::kEpiCols) {
#pragma unroll 1
        for (int cc = 0; cc < C::kEpiCols; cc += 16) {
          uint32_t v[16];
          tc_ld16(t_acc + c0 + cc, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) mine[(cc + j) * C::kEpiRowFloats] = __uint_as_float(v[j]);
        }
        if (c0 + C::kEpiCols >= BM) {
          tc_fence_before();
          mbar_arrive(smem_u32(&bar_tempty[acc]));
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (MODE == 1) {
          // one thread = one (token, 32-column group): SwiGLU-OAI, block maximum, E8M0 scale, 32 E4M3 codes
          for (int item = et; item < 2 * C::kEpiCols; item += 128) {
            const int j = item >> 1, g = item & 1;
            const float4* src = reinterpret_cast<const float4*>(stage_f + j * C::kEpiRowFloats + g * 68);
            float h[32];
            float amax = 0.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float4 gv = src[k], uv = src[8 + k];
              h[4 * k + 0] = swiglu_oai(gv.x, uv.x);
              h[4 * k + 1] = swiglu_oai(gv.y, uv.y);
              h[4 * k + 2] = swiglu_oai(gv.z, uv.z);
              h[4 * k + 3] = swiglu_oai(gv.w, uv.w);
            }
#pragma unroll
            for (int k = 0; k < 32; ++k) amax = fmaxf(amax, fabsf(h[k]));
            const int sc = mxfp8_scale(amax);
            const float inv = __uint_as_float(static_cast<uint32_t>(254 - sc) << 23);
            uint32_t words[8];
#pragma unroll
            for (int wd = 0; wd < 8; ++wd)
              words[wd] = cvt_e4m3x2(h[4 * wd] * inv, h[4 * wd + 1] * inv) |
                          (cvt_e4m3x2(h[4 * wd + 2] * inv, h[4 * wd + 3] * inv) << 16);
            const int grp = 2 * mt + g, n = c0 + j;
            uint4* dst = reinterpret_cast<uint4*>(ep.h8 + (row0 + n) * kI + grp * 32);
            dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
            dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
            ep.sfh8[(static_cast<int64_t>(b) * kS2TilesK + (grp >> 2)) * kAtomBytes + atom_offset(n, grp & 3)] =
                static_cast<uint8_t>(sc);
          }
        } else {
          // a warp writes one token's 128 output columns as 256 contiguous bytes
          for (int item = et; item < C::kEpiCols * 32; item += 128) {
            const int j = item >> 5, seg = item & 31;
            const int64_t row = row0 + c0 + j;
            if (row < ep.tokens) {
              const float4 x4 = *reinterpret_cast<const float4*>(stage_f + j * C::kEpiRowFloats + seg * 4);
              const __nv_bfloat162 lo = __floats2bfloat162_rn(x4.x, x4.y);
              const __nv_bfloat162 hi = __floats2bfloat162_rn(x4.z, x4.w);
              uint2 packed;
              packed.x = *reinterpret_cast<const uint32_t*>(&lo);
              packed.y = *reinterpret_cast<const uint32_t*>(&hi);
              *reinterpret_cast<uint2*>(ep.out + row * kH + mt * 128 + seg * 4) = packed;
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
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

template <int MODE, int BM>
static int launch_shared(const CUtensorMap& mx, const uint8_t* w_tiles, const uint8_t* sf_x, int n_blocks,
                         const SharedEpilogue& ep, int32_t* status, cudaStream_t stream) {
  using C = Cfg8<MODE, BM>;
  static PerDeviceOnce once;
  const int rc = once.run([] {
    return static_cast<int>(cudaFuncSetAttribute(shared_gemm_kernel<MODE, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 C::kSmemBytes));
  });
  if (rc) return rc;
  const int units = n_blocks * C::kTilesM;
  const int grid = units < sm_count() ? units : sm_count();
  if (grid <= 0) return 0;
  B200MOE_LAUNCH((shared_gemm_kernel<MODE, BM>), grid, 224, C::kSmemBytes, stream, mx, w_tiles, sf_x, n_blocks, ep, status);
  return 0;
}

template <int MODE>
static int launch_shared_bm(int bm, const CUtensorMap& mx, const uint8_t* w_tiles, const uint8_t* sf_x, int n_blocks,
                            const SharedEpilogue& ep, int32_t* status, cudaStream_t stream) {
  switch (bm) {
    case 16: return launch_shared<MODE, 16>(mx, w_tiles, sf_x, n_blocks, ep, status, stream);
    case 32: return launch_shared<MODE, 32>(mx, w_tiles, sf_x, n_blocks, ep, status, stream);
    case 64: return launch_shared<MODE, 64>(mx, w_tiles, sf_x, n_blocks, ep, status, stream);
    case 128: return launch_shared<MODE, 128>(mx, w_tiles, sf_x, n_blocks, ep, status, stream);
  }
  return B200MOE_E_ARG;
}

static size_t up1k(size_t v) { return (v + 1023) / 1024 * 1024; }

struct SharedWorkspace {
  uint8_t *x8, *sfx8, *h8, *sfh8;
  size_t bytes;
  int bm;
  int64_t rows;
};

static SharedWorkspace carve_shared(uint8_t* base, int64_t tokens) {
  SharedWorkspace ws{};
  ws.bm = b200moe_shared_block_rows(tokens);
  ws.rows = (tokens + ws.bm - 1) / ws.bm * ws.bm;
  const size_t blocks = static_cast<size_t>(ws.rows / ws.bm);
  size_t off = 0;
  auto take = [&](size_t n) {
    uint8_t* p = base ? base + off : nullptr;
    off = up1k(off + n);
    return p;
  };
  ws.x8 = take(ws.rows * kH);
  ws.sfx8 = take(blocks * kS1TilesK * kAtomBytes);
  ws.h8 = take(ws.rows * kI);
  ws.sfh8 = take(blocks * kS2TilesK * kAtomBytes);
  ws.bytes = off;
  return ws;
}

int set_wait_limit_shared(unsigned long long ns) { return set_wait_limit_here(ns); }

}  // namespace b200moe

// Dense blocks: the widest block that the token count fills, so the 14 MB of weights are streamed as few times as
// possible (once up to 128 tokens) and the few CTAs this takes leave the other SMs to the routed experts' kernels.
extern "C" int b200moe_shared_block_rows(int64_t tokens) {
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS) return 0;
  return tokens <= 16 ? 16 : tokens <= 32 ? 32 : tokens <= 64 ? 64 : 128;
}

extern "C" int b200moe_preshuffle_shared(const uint8_t* w13, const uint8_t* s13, const uint8_t* w2, const uint8_t* s2,
                                         uint8_t* w13t, uint8_t* w2t, void* stream) {
  using namespace b200moe;
  if (!w13 || !s13 || !w2 || !s2 || !w13t || !w2t) return B200MOE_E_ARG;
  if (misaligned(w13, 16) || misaligned(w2, 16) || misaligned(w13t, 16) || misaligned(w2t, 16)) return B200MOE_E_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200MOE_LAUNCH_PLAIN((preshuffle_shared_kernel<kH, kW13Tiles, true>), dim3(128, kW13Tiles), 128, 0, st, w13, s13, w13t);
  B200MOE_LAUNCH_PLAIN((preshuffle_shared_kernel<kI, kW2Tiles, false>), dim3(128, kW2Tiles), 64, 0, st, w2, s2, w2t);
  return 0;
}

extern "C" size_t b200moe_shared_workspace_bytes(int64_t tokens) {
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS) return 0;
  return b200moe::carve_shared(nullptr, tokens).bytes;
}

extern "C" int b200moe_shared_quant(const void* x_bf16, int64_t tokens, int bm, uint8_t* codes8, uint8_t* atoms,
                                    void* stream) {
  using namespace b200moe;
  if (!x_bf16 || !codes8 || !atoms || tokens < 1 || tokens > B200MOE_MAX_TOKENS) return B200MOE_E_ARG;
  const int shift = bm == 16 ? 4 : bm == 32 ? 5 : bm == 64 ? 6 : bm == 128 ? 7 : -1;
  if (shift < 0) return B200MOE_E_ARG;
  if (misaligned(x_bf16, 16) || misaligned(codes8, 16) || misaligned(atoms, 16)) return B200MOE_E_ALIGN;
  const int64_t rows = (tokens + bm - 1) / bm * bm;
  B200MOE_LAUNCH(shared_quant_kernel, static_cast<unsigned>(rows), 256, 0, static_cast<cudaStream_t>(stream),
                 static_cast<const uint4*>(x_bf16), tokens, shift, codes8, atoms, static_cast<uint8_t*>(nullptr));
  return 0;
}

extern "C" int b200moe_shared_quant_rows(const void* x_bf16, int64_t tokens, uint8_t* codes8, uint8_t* scales,
                                         void* stream) {
  using namespace b200moe;
  if (!x_bf16 || !codes8 || !scales || tokens < 1 || tokens > B200MOE_MAX_TOKENS) return B200MOE_E_ARG;
  if (misaligned(x_bf16, 16) || misaligned(codes8, 16) || misaligned(scales, 4)) return B200MOE_E_ALIGN;
  B200MOE_LAUNCH(shared_quant_kernel, static_cast<unsigned>(tokens), 256, 0, static_cast<cudaStream_t>(stream),
                 static_cast<const uint4*>(x_bf16), tokens, 4, codes8, static_cast<uint8_t*>(nullptr), scales);
  return 0;
}

static int shared_gemms(const uint8_t* w13t, const uint8_t* w2t, const uint8_t* codes8, int64_t code_rows,
                        const b200moe::SharedWorkspace& ws, void* out_bf16, int64_t tokens, int32_t* status, void* stream) {
  using namespace b200moe;
  const int n_blocks = static_cast<int>(ws.rows / ws.bm);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap mx, mh;
  int r;
  // code_rows may be the unpadded token count: boxes that reach beyond it read zeros
  if ((r = make_map(&mx, codes8, kH, static_cast<uint64_t>(code_rows), static_cast<uint32_t>(ws.bm)))) return r;
  if ((r = make_map(&mh, ws.h8, kI, static_cast<uint64_t>(ws.rows), static_cast<uint32_t>(ws.bm)))) return r;
  SharedEpilogue ep{};
  ep.h8 = ws.h8;
  ep.sfh8 = ws.sfh8;
  ep.out = static_cast<__nv_bfloat16*>(out_bf16);
  ep.tokens = tokens;
  if ((r = launch_shared_bm<1>(ws.bm, mx, w13t, ws.sfx8, n_blocks, ep, status, st))) return r;
  return launch_shared_bm<2>(ws.bm, mh, w2t, ws.sfh8, n_blocks, ep, status, st);
}

extern "C" int b200moe_shared_expert(const uint8_t* w13t, const uint8_t* w2t, const void* x_bf16, int64_t tokens,
                                     void* workspace, size_t workspace_bytes, void* out_bf16, int32_t* status,
                                     void* stream) {
  using namespace b200moe;
  if (!w13t || !w2t || !x_bf16 || !workspace || !out_bf16 || !status) return B200MOE_E_ARG;
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS) return B200MOE_E_ARG;
  if (misaligned(workspace, 256) || misaligned(w13t, 16) || misaligned(w2t, 16) || misaligned(out_bf16, 16))
    return B200MOE_E_ALIGN;
  SharedWorkspace ws = carve_shared(static_cast<uint8_t*>(workspace), tokens);
  if (workspace_bytes < ws.bytes) return B200MOE_E_ARG;
  const int r = b200moe_shared_quant(x_bf16, tokens, ws.bm, ws.x8, ws.sfx8, stream);
  if (r) return r;
  return shared_gemms(w13t, w2t, ws.x8, ws.rows, ws, out_bf16, tokens, status, stream);
}

extern "C" int b200moe_scales_to_atoms(const uint8_t* rows, int64_t tokens, int cols, int bm, uint8_t* atoms, void* stream);

extern "C" int b200moe_shared_expert_quantized(const uint8_t* w13t, const uint8_t* w2t, const uint8_t* codes8,
                                               const uint8_t* scales, int64_t tokens, void* workspace,
                                               size_t workspace_bytes, void* out_bf16, int32_t* status, void* stream) {
  using namespace b200moe;
  if (!w13t || !w2t || !codes8 || !scales || !workspace || !out_bf16 || !status) return B200MOE_E_ARG;
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS) return B200MOE_E_ARG;
  if (misaligned(workspace, 256) || misaligned(w13t, 16) || misaligned(w2t, 16) || misaligned(out_bf16, 16) ||
      misaligned(codes8, 16) || misaligned(scales, 4))
    return B200MOE_E_ALIGN;
  SharedWorkspace ws = carve_shared(static_cast<uint8_t*>(workspace), tokens);
  if (workspace_bytes < ws.bytes) return B200MOE_E_ARG;
  const int r = b200moe_scales_to_atoms(scales, tokens, kH / 32, ws.bm, ws.sfx8, stream);
  if (r) return r;
  return shared_gemms(w13t, w2t, codes8, tokens, ws, out_bf16, tokens, status, stream);
}
