// Prefill GEMM1 (+ SwiGLU-OAI + MXFP4 requantisation) on CTA PAIRS: a cluster of two CTAs on neighbouring SMs runs one
// tcgen05.mma.cta_group::2 of M = 256 token rows x N = 256 weight rows x K = 64 per instruction.
//
// Why pairs. With one CTA per tile (128 x 128 per MMA) every 64 cycles of tensor math read 8 KB of operands from shared
// memory, and the same bytes were written there by the copy engine just before: shared memory moves 128 bytes per cycle
// and is the limit (tensor pipe measured 50 % busy). In a pair each CTA holds its own 128 token rows (its half of A) and
// 128 of the 256 weight rows (its half of B); the hardware hands each B half to the partner, so per 512 cycles of math a
// CTA writes 34 KB and reads 32 KB instead of 68 + 64.
//
// Work. The routing sort (block height 128) lays an expert's row blocks next to one another. A unit is (two consecutive
// blocks of one expert, or its last odd block alone) x (a pair of W13 tiles = 128 intermediate columns, gate and up). CTA
// r of the pair loads the tokens of block b0 + r and weight tile 2*tp + r; both load the 1 KB of scales of both tiles.
// With a single block the second CTA still supplies its weight half but has no rows of its own.
//
//   warp 0     producer (both CTAs): TMA tile loads, all completing on the LEADER's (CTA 0) full barrier
//   warp 1     allocates / frees tensor memory (both CTAs); in the leader one thread issues the MMAs for both
//   warps 2, 11 leader: one thread each copies half of the stage's scales into tensor memory in both CTAs
//              (tcgen05.cp.cta_group::2); two threads because every tcgen05 instruction costs its thread ~60 cycles
//   warps 3-10 epilogue (both CTAs): thread = one token row (TMEM lane), everything in registers; the accumulator is
//              handed back as soon as it sits in registers, so the next unit's MMAs run under the epilogue's arithmetic
//
// No load is a multicast load; stage release and accumulator hand-over use one plain tcgen05.commit per CTA. Every wait
// is bounded as in the other kernels (status word B200MOE_DEV_TIMEOUT, drain, free, return).
#include <cuda.h>

#include "tc_host.cuh"
#include "tc_ptx.cuh"

namespace b200moe {

struct PairCfg {
  static constexpr int kStages = 6;
  static constexpr int kTokOff = 0;                 // this CTA's 128 token rows x 128 bytes (128-byte swizzle)
  static constexpr int kWOff = 128 * 128;           // this CTA's 128 weight rows x 128 bytes (tile record image)
  static constexpr int kSfTokOff = 2 * 128 * 128;   // token scales: two atoms
  static constexpr int kSfWLoOff = kSfTokOff + 2 * kAtomBytes;   // scales of tile 2*tp (weight rows 0..127 of N)
  static constexpr int kSfWHiOff = kSfWLoOff + 2 * kAtomBytes;   // scales of tile 2*tp+1 (rows 128..255)
  static constexpr int kStageBytes = kSfWHiOff + 2 * kAtomBytes; // 35840
  static constexpr int kThreads = 32 * 12;
  static constexpr int kAccCols = 256;
  static constexpr int kSfSets = 8;                 // >= kStages; a set: 8 token-scale columns + 16 weight-scale columns
  static constexpr int kSfCol = kAccCols;
  static constexpr int kTmemCols = 512;
  static constexpr int kMaxBlocks = 2880;           // row blocks of 128 at the largest token count the library accepts
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
  static constexpr int kTilePairs = kW13Tiles / 2;
  static constexpr uint32_t kWeightTx = 128 * 128 + 4 * kAtomBytes;   // per CTA: codes + both tiles' scales
  static constexpr uint32_t kTokenTx = 128 * 128 + 2 * kAtomBytes;    // per CTA that has a row block
};
static_assert(PairCfg::kSfCol + 24 * PairCfg::kSfSets <= PairCfg::kTmemCols, "tensor memory columns");
static_assert(kW13Tiles % 2 == 0, "W13 tiles come in pairs");

// ------------------------------------------------------------------------------------------------ PTX, pair forms
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tile load whose bytes are counted on a barrier that may sit in the partner CTA (`bar` is a shared::cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
          "r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tc_cp_scales_pair(uint32_t taddr, uint32_t desc_lo) {
  asm volatile("{\n.reg .b64 d;\nmov.b64 d, {%1, %2};\ntcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d;\n}\n" ::"r"(taddr),
               "r"(desc_lo), "n"(kScaleDescHi)
               : "memory");
}
__device__ __forceinline__ void tc_mma_mxf4_pair(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t sfa,
                                                 uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .b64 da, db;\n.reg .pred p;\nmov.b64 da, {%1, %7};\nmov.b64 db, {%2, %7};\nsetp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %3, [%4], [%5], p;\n}\n" ::"r"(d),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate), "n"(kOperandDescHi)
      : "memory");
}
__device__ __forceinline__ void drain_tcgen05_pair(uint32_t bar) {
  tc_commit_pair(bar);
  const uint64_t t0 = global_timer(), limit = wait_limit_ns();
  while (!mbar_try_wait(bar, 0) && global_timer() - t0 < limit) {}
}

// One (token row, 32-column group of the intermediate): SwiGLU-OAI of the 32 gate / up accumulators, the block maximum, the
// E8M0 byte and the 32 E2M1 codes -> one 16-byte store of codes and one scale byte; everything thread-local.
__device__ __forceinline__ void swiglu_quant_store(const uint32_t (&gv)[32], const uint32_t (&uv)[32], uint8_t* hq,
                                                   uint8_t* sfh, int64_t row, int b, int tr, int grp) {
  float h[32];
  float amax = 0.0f;
#pragma unroll
  for (int k = 0; k < 32; ++k) {
    h[k] = swiglu_oai(__uint_as_float(gv[k]), __uint_as_float(uv[k]));
    amax = fmaxf(amax, fabsf(h[k]));
  }
  const int sc = quark_even_e8m0(amax);
  const float inv = __uint_as_float(static_cast<uint32_t>(254 - sc) << 23);
  uint32_t words[4];
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    uint32_t acc_w = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) acc_w |= cvt_e2m1x2(h[8 * wd + 2 * k] * inv, h[8 * wd + 2 * k + 1] * inv) << (8 * k);
    words[wd] = acc_w;
  }
  *reinterpret_cast<uint4*>(hq + row * (kI / 2) + grp * 16) = make_uint4(words[0], words[1], words[2], words[3]);
  sfh[(static_cast<int64_t>(b) * (kI / 128) + (grp >> 2)) * kAtomBytes + atom_offset(tr, grp & 3)] = static_cast<uint8_t>(sc);
}

// what a row block is to the pair schedule
enum : uint8_t { kBlockSkip = 0, kBlockSingle = 1, kBlockPair = 2 };

// ------------------------------------------------------------------------------------------------ kernel
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PairCfg::kThreads, 1)
    gemm1_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_sfx,
                      const __grid_constant__ CUtensorMap map_wc, const __grid_constant__ CUtensorMap map_ws,
                      const int32_t* __restrict__ block_expert, const int32_t* __restrict__ num_valid,
                      uint8_t* __restrict__ hq, uint8_t* __restrict__ sfh, int32_t* status, int num_experts,
                      int max_blocks) {
  using C = PairCfg;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[C::kStages];   // used in the leader: both CTAs' bytes of the stage have landed
  __shared__ __align__(8) uint64_t bar_empty[C::kStages];  // in each CTA: the MMAs that read the stage have completed
  __shared__ __align__(8) uint64_t bar_sf[C::kStages];     // leader: the stage's scales are in tensor memory
  __shared__ __align__(8) uint64_t bar_tfull;              // in each CTA: the unit's accumulator is complete
  __shared__ __align__(8) uint64_t bar_tempty;             // leader: both CTAs' epilogues have read the accumulator
  __shared__ __align__(8) uint64_t bar_drain[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ uint8_t s_kind[C::kMaxBlocks];
  __shared__ uint16_t s_unit[C::kMaxBlocks];  // the blocks that start a unit, in order: block | pair << 15
  __shared__ int s_count[C::kThreads + 1];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile int* abort_v = &abort_flag;
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
      mbar_init(smem_u32(&bar_sf[s]), 2);  // the two scale-copy threads
    }
    mbar_init(smem_u32(&bar_tfull), 1);
    mbar_init(smem_u32(&bar_tempty), 16);  // one arrival per epilogue warp of both CTAs
    mbar_init(smem_u32(&bar_drain[0]), 1);
    mbar_init(smem_u32(&bar_drain[1]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(static_cast<uint32_t>(C::kTmemCols))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  pdl_wait();
  launder(block_expert);
  launder(num_valid);
  int n_blocks = __ldcg(num_valid) / 128;
  if (n_blocks < 0 || n_blocks > max_blocks || n_blocks > C::kMaxBlocks) {
    if (threadIdx.x == 0) atomicExch(status, B200MOE_DEV_BAD_INDEX);
    n_blocks = 0;
  }
  // Pair schedule: a block at an even position inside its expert starts a unit (with its successor when that belongs to
  // the same expert); a block at an odd position is covered by its predecessor's unit.
  for (int b = threadIdx.x; b < n_blocks; b += C::kThreads) {
    const int e = __ldcg(block_expert + b);
    int pos = 0;
    while (b - 1 - pos >= 0 && __ldcg(block_expert + b - 1 - pos) == e) ++pos;
    uint8_t kind = kBlockSkip;
    if ((pos & 1) == 0) kind = (b + 1 < n_blocks && __ldcg(block_expert + b + 1) == e) ? kBlockPair : kBlockSingle;
    if (e < 0 || e >= num_experts) {  // never form an address from an expert id outside the weights
      atomicExch(status, B200MOE_DEV_BAD_INDEX);
      kind = kBlockSkip;
    }
    s_kind[b] = kind;
  }
  __syncthreads();
  // The units in order, so that they can be dealt evenly: every thread counts the unit-starting blocks of its contiguous
  // chunk, one thread turns the counts into offsets, every thread writes its chunk's entries.
  {
    const int chunk = (n_blocks + C::kThreads - 1) / C::kThreads;
    const int lo = min(n_blocks, static_cast<int>(threadIdx.x) * chunk), hi = min(n_blocks, lo + chunk);
    int cnt = 0;
    for (int b = lo; b < hi; ++b) cnt += s_kind[b] != kBlockSkip;
    s_count[threadIdx.x] = cnt;
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      for (int i = 0; i < C::kThreads; ++i) {
        const int c = s_count[i];
        s_count[i] = run;
        run += c;
      }
      s_count[C::kThreads] = run;
    }
    __syncthreads();
    int pos = s_count[threadIdx.x];
    for (int b = lo; b < hi; ++b)
      if (s_kind[b] != kBlockSkip) s_unit[pos++] = static_cast<uint16_t>(b | (s_kind[b] == kBlockPair ? 0x8000 : 0));
  }
  __syncthreads();
  const int n_clusters = static_cast<int>(gridDim.x >> 1), cluster = static_cast<int>(blockIdx.x >> 1);
  const int total = s_count[C::kThreads] * C::kTilePairs;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer (both CTAs)
    if (lane == 0) {
      const uint32_t full0 = map_to_cta(smem_u32(&bar_full[0]), 0);  // the leader's barriers, as seen from this CTA
      uint32_t it = 0;
      bool ok = true;
      for (int u = cluster; u < total && ok; u += n_clusters) {
        const uint32_t ub = s_unit[u / C::kTilePairs];
        const int b0 = static_cast<int>(ub & 0x7fffu), tp = u % C::kTilePairs;
        const bool pair = (ub & 0x8000u) != 0;
        const bool have_rows = leader || pair;
        const int e = __ldcg(block_expert + b0);
        const int my_block = b0 + static_cast<int>(rank);
        // rows of the weight matrix seen as [records * 136][128 bytes]: 128 rows of codes, then 8 rows of scales
        const int rec_mine = ((e * kW13Tiles + 2 * tp + static_cast<int>(rank)) * kK1Tiles) * 136;
        const int rec_lo = ((e * kW13Tiles + 2 * tp) * kK1Tiles) * 136, rec_hi = rec_lo + kK1Tiles * 136;
        for (int kt = 0; kt < kK1Tiles; ++kt, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_v, status)) { ok = false; break; }
          const uint32_t full = full0 + 8u * s, base = tiles + s * C::kStageBytes;
          if (leader)
            mbar_arrive_expect_tx(smem_u32(&bar_full[s]),
                                  2u * C::kWeightTx + (pair ? 2u : 1u) * C::kTokenTx);
          tma_load_2d_pair(base + C::kWOff, &map_wc, 0, rec_mine + kt * 136, full);
          tma_load_2d_pair(base + C::kSfWLoOff, &map_ws, 0, rec_lo + kt * 136 + 128, full);
          tma_load_2d_pair(base + C::kSfWHiOff, &map_ws, 0, rec_hi + kt * 136 + 128, full);
          if (have_rows) {
            tma_load_2d_pair(base + C::kTokOff, &map_x, kt * 128, my_block * 128, full);
            tma_load_2d_pair(base + C::kSfTokOff, &map_sfx, 0, (my_block * (kH / 128) + 2 * kt) * 4, full);
          }
        }
      }
      if (!ok && leader) drain_copies(bar_full, it, C::kStages);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue (leader only)
    if (lane == 0 && leader) {
      // E2M1 x E2M1, UE8M0 scales, M = 256 (128 token rows per CTA), N = 256 weight rows
      constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(256 >> 3) << 17) | (1u << 23) |
                                  (static_cast<uint32_t>(256 >> 4) << 24);
      constexpr uint32_t kId0 = kIdesc, kId1 = kIdesc | (2u << 29) | (2u << 4);
      const uint32_t empty_peer0 = map_to_cta(smem_u32(&bar_empty[0]), 1), tfull_peer = map_to_cta(smem_u32(&bar_tfull), 1);
      uint32_t it = 0, ui = 0;
      bool ok = true;
      for (int u = cluster; u < total && ok; u += n_clusters) {
        if (!mbar_wait(smem_u32(&bar_tempty), (ui & 1u) ^ 1u, abort_v, status)) break;
        tc_fence_after();
        for (int kt = 0; kt < kK1Tiles; ++kt, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u, sfset = it & (C::kSfSets - 1);
          if (!mbar_wait(smem_u32(&bar_sf[s]), ph, abort_v, status)) { ok = false; break; }
          tc_fence_after();  // rows written by plain copies
          const uint32_t lo = (tiles + s * C::kStageBytes) >> 4;
          const uint32_t x_lo = lo + (C::kTokOff >> 4), w_lo = lo + (C::kWOff >> 4);
          const uint32_t t_sft = tmem_base + C::kSfCol + 24u * sfset, t_sfw = t_sft + 8u;
          // 64 K-elements = 32 bytes per MMA; scale bytes {0,1} or {2,3} of the K-atom's cells
          tc_mma_mxf4_pair(tmem_base, x_lo, w_lo, kId0, t_sft, t_sfw, static_cast<uint32_t>(kt != 0));
          tc_mma_mxf4_pair(tmem_base, x_lo + 2, w_lo + 2, kId1, t_sft, t_sfw, 1u);
          tc_mma_mxf4_pair(tmem_base, x_lo + 4, w_lo + 4, kId0, t_sft + 4, t_sfw + 8, 1u);
          tc_mma_mxf4_pair(tmem_base, x_lo + 6, w_lo + 6, kId1, t_sft + 4, t_sfw + 8, 1u);
          tc_commit_pair(smem_u32(&bar_empty[s]));  // the stage is free again, in this CTA ...
          tc_commit_pair(empty_peer0 + 8u * s);     // ... and in the partner
        }
        if (ok) {
          tc_commit_pair(smem_u32(&bar_tfull));
          tc_commit_pair(tfull_peer);
        }
        ++ui;
      }
      if (*abort_v) drain_tcgen05_pair(smem_u32(&bar_drain[0]));
    }
  } else if (warp == 2 || warp == 11) {
    // ---------------------------------------------------------------- scale copies into both CTAs' tensor memory (leader)
    // warp 2: the token scales and the first K-atom's weight scales of rows 0..127; warp 11: the other three atoms
    if (lane == 0 && leader) {
      const bool first = warp == 2;
      uint32_t it = 0;
      bool ok = true;
      for (int u = cluster; u < total && ok; u += n_clusters) {
        for (int kt = 0; kt < kK1Tiles; ++kt, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u, sfset = it & (C::kSfSets - 1);
          if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_v, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t lo = (tiles + s * C::kStageBytes) >> 4;
          const uint32_t t_sft = tmem_base + C::kSfCol + 24u * sfset, t_sfw = t_sft + 8u;
          // token scales: K-atom 0, K-atom 1 (each CTA its own rows); weight scales per K-atom: rows 0..127, rows 128..255
          if (first) {
            tc_cp_scales_pair(t_sft, lo + (C::kSfTokOff >> 4));
            tc_cp_scales_pair(t_sft + 4, lo + ((C::kSfTokOff + kAtomBytes) >> 4));
            tc_cp_scales_pair(t_sfw, lo + (C::kSfWLoOff >> 4));
          } else {
            tc_cp_scales_pair(t_sfw + 4, lo + (C::kSfWHiOff >> 4));
            tc_cp_scales_pair(t_sfw + 8, lo + ((C::kSfWLoOff + kAtomBytes) >> 4));
            tc_cp_scales_pair(t_sfw + 12, lo + ((C::kSfWHiOff + kAtomBytes) >> 4));
          }
          tc_commit_pair(smem_u32(&bar_sf[s]));
        }
      }
      if (*abort_v) drain_tcgen05_pair(smem_u32(&bar_drain[1]));
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs, warps 3..10)
    const int q = warp & 3;                 // the TMEM lane quarter this warp may read
    const int half = ((warp - 3) >> 2) & 1; // which 128 of the 256 accumulator columns (= which W13 tile of the pair)
    const int tr = q * 32 + lane;           // token row inside the block = TMEM lane
    const uint32_t tempty_leader = map_to_cta(smem_u32(&bar_tempty), 0);
    uint32_t ui = 0;
    for (int u = cluster; u < total; u += n_clusters) {
      const uint32_t ub = s_unit[u / C::kTilePairs];
      const int b0 = static_cast<int>(ub & 0x7fffu), tp = u % C::kTilePairs;
      const bool have_rows = leader || (ub & 0x8000u) != 0;
      const int b = b0 + static_cast<int>(rank);
      const int64_t row = static_cast<int64_t>(b) * 128 + tr;
      // the warp decides together: tcgen05.ld below needs all 32 lanes
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_tfull), ui & 1u, abort_v, status))) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + 128u * half + (static_cast<uint32_t>(q * 32) << 16);
      // columns of a tile: [gate 32 | up 32 | gate 32 | up 32] of 64 intermediate columns. All 128 values of this thread
      // go to registers first, then the accumulator is handed back (one arrival per warp, on the leader's barrier): the
      // next unit's MMAs run while SwiGLU, the block maxima and the codes are computed, all thread-local.
      uint32_t acc[4][32];
      if (have_rows) {
        tc_ld32_nowait(t_acc, acc[0]);
        tc_ld32_nowait(t_acc + 32, acc[1]);
        tc_ld32_nowait(t_acc + 64, acc[2]);
        tc_ld32_nowait(t_acc + 96, acc[3]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader);
      ++ui;
      if (!have_rows) continue;
#pragma unroll
      for (int g = 0; g < 2; ++g)
        swiglu_quant_store(acc[2 * g], acc[2 * g + 1], hq, sfh, row, b, tr, 4 * tp + 2 * half + g);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees tensor memory or leaves while the partner may still signal or read it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(C::kTmemCols))
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ one CTA, N = 256
// The same 256-column unit on ONE CTA: M = 128 token rows (one row block) x N = 256 weight rows (two W13 tiles) per
// tcgen05.mma.cta_group::1. Every block is a unit, so an expert's odd last block costs nothing extra; the price is that the
// CTA stages both weight tiles itself (48 KB of codes per stage, 4 stages).
//
// Two rings. Measured on the one-ring form of this kernel (codes and scales of a K-tile in one stage): a stage's ring was
// free -> 6 copies issued (~650 cycles) -> last byte landed (~1350) -> scales copied to tensor memory and seen by the MMA
// thread (~860) -> MMAs run and seen complete (~680), 3500 cycles for 4 stages = 880 per stage against 512 of tensor time.
// The scales are 6 % of the bytes, so they get a ring of their own, twice as deep: a dedicated warp fetches them 8 K-tiles
// ahead and the two copy threads move them into tensor memory as soon as the stage 4 tiles back has been consumed, which
// is long before the codes of their own tile land. The MMA thread then waits for codes only, and the scale copy has left
// the critical ring.
//
//   warp 0      code producer: TMA of the two weight tiles (and, sorted input, the token tile)
//   warp 1      tensor memory; one thread issues the MMAs
//   warps 2, 3  one thread each: three of the six scale atoms smem -> tensor memory (tcgen05.cp), then commit
//   warps 4-7   GATHER only: each fetches 32 token rows of the block by the sorted list (16-byte asynchronous copies)
//   warp 8      scale producer: TMA of the weight scales (and the token scales, or GATHER: gathers them, 4 rows per lane)
//   warps 12-19 epilogue: thread = one token row, a whole accumulator half-row in registers
// 20 warps start with 96 registers; warps 0..11 drop to 48 and the epilogue warps rise to 168
// (setmaxnreg; 12 x 48 + 8 x 168 = 20 x 96: the exchange must balance inside what the CTA was given at launch).
struct WideCfg {
  static constexpr int kStages = 4;                  // code ring
  static constexpr int kSfStages = 8;                // scale ring = scale sets in tensor memory
  static constexpr int kTokOff = 0;
  static constexpr int kWOff = 128 * 128;            // 256 weight rows x 128 bytes: tile 2*tp, then tile 2*tp+1
  static constexpr int kStageBytes = 3 * 128 * 128;  // 49152
  static constexpr int kSfRingOff = kStages * kStageBytes;
  static constexpr int kSfTokOff = 0;                // inside a scale slot: token atoms 0, 1
  static constexpr int kSfWLoOff = 2 * kAtomBytes;   // tile 2*tp, K-atoms 0, 1
  static constexpr int kSfWHiOff = 4 * kAtomBytes;   // tile 2*tp+1
  static constexpr int kSfSlotBytes = 6 * kAtomBytes;
  static constexpr int kThreads = 32 * 20;
  static constexpr int kGather0 = 4, kScaleProducer = 8, kEpilogue0 = 12;
  static constexpr int kSfCol = 256;
  static constexpr int kTmemCols = 512;
  static constexpr int kSmemBytes = kSfRingOff + kSfStages * kSfSlotBytes + 1024;
  static constexpr int kTilePairs = kW13Tiles / 2;
};
static_assert(WideCfg::kSfCol + 24 * WideCfg::kSfStages <= WideCfg::kTmemCols, "tensor memory columns");
static_assert(kK1Tiles % WideCfg::kSfStages == 0, "a unit starts at slot 0 of both rings");

__device__ __forceinline__ void tc_mma_mxf4_wide(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t sfa,
                                                 uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .b64 da, db;\n.reg .pred p;\nmov.b64 da, {%1, %7};\nmov.b64 db, {%2, %7};\nsetp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %3, [%4], [%5], p;\n}\n" ::"r"(d),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate), "n"(kOperandDescHi)
      : "memory");
}

// Token rows in their unsorted, row-major quantised form (what the row quantiser writes) plus the sorted (token, slot)
// list: with these the kernel gathers its 128 token rows itself and no sorted copy of the activations exists.
struct GatherRows {
  const uint8_t* codes;       // [tokens][kH / 2]
  const uint8_t* scales;      // [tokens][kH / 32]
  const int32_t* sorted_ids;  // token | slot << 24; a token index >= tokens marks a padding row
  int64_t tokens;
  int by_pair;                // 1: codes / scales hold one row per (token, slot) pair, row 4 * token + slot
};

// row of the quantised input that sorted entry `sid` reads, ~0 for a padding row
__device__ __forceinline__ uint32_t gather_row(int sid, const GatherRows& rows) {
  const uint32_t tok = static_cast<uint32_t>(sid) & 0x00ffffffu;
  if (tok >= rows.tokens) return 0xffffffffu;
  return rows.by_pair ? tok * kTopK + ((static_cast<uint32_t>(sid) >> 24) & 3u) : tok;
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {  // arrives once this thread's copies so far have landed
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// GATHER false: the token rows arrive sorted (map_x, map_sfx). GATHER true: rows come from `rows` through the sorted list
// (a padding row is zero-filled), written in the 128-byte swizzle, the scale bytes into their atom cells.
template <bool GATHER>
__global__ void __launch_bounds__(WideCfg::kThreads, 1)
    gemm1_wide_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_sfx,
                      const __grid_constant__ CUtensorMap map_wc, const __grid_constant__ CUtensorMap map_ws,
                      const GatherRows rows, const int32_t* __restrict__ block_expert,
                      const int32_t* __restrict__ num_valid, uint8_t* __restrict__ hq, uint8_t* __restrict__ sfh,
                      int32_t* status, int num_experts, int max_blocks, const int32_t* __restrict__ block_range) {
  using C = WideCfg;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[C::kStages];     // the stage's codes have landed
  __shared__ __align__(8) uint64_t bar_empty[C::kStages];    // the MMAs that read the stage have completed
  __shared__ __align__(8) uint64_t bar_sfull[C::kSfStages];  // the slot's scales have landed in shared memory
  __shared__ __align__(8) uint64_t bar_sf[C::kSfStages];     // ... and have been copied to tensor memory
  __shared__ __align__(8) uint64_t bar_tfull;
  __shared__ __align__(8) uint64_t bar_tempty;
  __shared__ __align__(8) uint64_t bar_drain[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sf_ring = tiles + C::kSfRingOff;
  volatile int* abort_v = &abort_flag;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), GATHER ? 1 + 128 : 1);  // the TMA arrival (+ one per gathering lane)
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int j = 0; j < C::kSfStages; ++j) {
      mbar_init(smem_u32(&bar_sfull[j]), GATHER ? 1 + 32 : 1);
      mbar_init(smem_u32(&bar_sf[j]), 2);  // the two scale-copy threads
    }
    mbar_init(smem_u32(&bar_tfull), 1);
    mbar_init(smem_u32(&bar_tempty), 8);  // one arrival per epilogue warp
    mbar_init(smem_u32(&bar_drain[0]), 1);
    mbar_init(smem_u32(&bar_drain[1]), 1);
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
  launder(block_expert);
  launder(num_valid);
  int n_blocks = __ldcg(num_valid) / 128;
  if (n_blocks < 0 || n_blocks > max_blocks) {
    if (threadIdx.x == 0) atomicExch(status, B200MOE_DEV_BAD_INDEX);
    n_blocks = 0;
  }
  // `block_range` (may be null): the launch covers the row blocks [range[0], range[1]) only (a caller that splits the row
  // blocks into chunks, so that a following kernel can start on one chunk while this one works on the next)
  int b_lo = 0;
  if (block_range != nullptr) {
    launder(block_range);
    b_lo = max(0, min(__ldcg(block_range), n_blocks));
    n_blocks = max(b_lo, min(__ldcg(block_range + 1), n_blocks)) - b_lo;
  }
  const int total = n_blocks * C::kTilePairs, stride = static_cast<int>(gridDim.x), first = static_cast<int>(blockIdx.x);
  const int32_t* sorted_ids = rows.sorted_ids;
  launder(sorted_ids);

  // The two register groups (three and two whole warpgroups) do not meet again before the kernel's last lines.
  if (warp < C::kEpilogue0) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
  if (warp == 0) {
    // ---------------------------------------------------------------- code producer (TMA)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int u = first; u < total && ok; u += stride) {
        const int b = b_lo + u / C::kTilePairs, tp = u % C::kTilePairs;
        int e = __ldcg(block_expert + b);
        if (e < 0 || e >= num_experts) {  // never form an address from an expert id outside the weights
          atomicExch(status, B200MOE_DEV_BAD_INDEX);
          e = 0;
        }
        // rows of the weight matrix seen as [records * 136][128 bytes]: 128 rows of codes, then 8 rows of scales
        const int rec_lo = ((e * kW13Tiles + 2 * tp) * kK1Tiles) * 136, rec_hi = rec_lo + kK1Tiles * 136;
        for (int kt = 0; kt < kK1Tiles; ++kt, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_v, status)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[s]), base = tiles + s * C::kStageBytes;
          mbar_arrive_expect_tx(full, (GATHER ? 2 : 3) * 128 * 128);
          tma_load_2d(base + C::kWOff, &map_wc, 0, rec_lo + kt * 136, full);
          tma_load_2d(base + C::kWOff + 128 * 128, &map_wc, 0, rec_hi + kt * 136, full);
          if (!GATHER) tma_load_2d(base + C::kTokOff, &map_x, kt * 128, b * 128, full);
        }
      }
      if (!ok) drain_copies(bar_full, it, C::kStages);
    }
  } else if (warp == C::kScaleProducer) {
    // ---------------------------------------------------------------- scale producer, 8 K-tiles deep
    // GATHER: lane L owns token rows L, L + 32, L + 64, L + 96 of the block: two 4-byte cells per row and K-tile
    const uint32_t cell = static_cast<uint32_t>(C::kSfTokOff + lane * 16);
    uint32_t it = 0;
    bool ok = true;
    for (int u = first; u < total && ok; u += stride) {
      const int b = b_lo + u / C::kTilePairs, tp = u % C::kTilePairs;
      int e = __ldcg(block_expert + b);
      if (e < 0 || e >= num_experts) e = 0;  // reported by the code producer
      const int rec_lo = ((e * kW13Tiles + 2 * tp) * kK1Tiles) * 136, rec_hi = rec_lo + kK1Tiles * 136;
      uint32_t soff[4];  // byte offset of the row's scales, ~0: a padding row
      if (GATHER) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const uint32_t row = gather_row(__ldcg(sorted_ids + b * 128 + 32 * m + lane), rows);
          soff[m] = row != 0xffffffffu ? row * static_cast<uint32_t>(kH / 32) : 0xffffffffu;
        }
      }
      for (int kt = 0; kt < kK1Tiles; ++kt, ++it) {
        const uint32_t j = it % C::kSfStages, ph = (it / C::kSfStages) & 1u;
        // the slot is free once the copy threads have moved its previous contents to tensor memory
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_sf[j]), ph ^ 1u, abort_v, status))) { ok = false; break; }
        const uint32_t sfull = smem_u32(&bar_sfull[j]), slot = sf_ring + j * C::kSfSlotBytes;
        if (lane == 0) {
          mbar_arrive_expect_tx(sfull, (GATHER ? 4 : 6) * kAtomBytes);
          tma_load_2d(slot + C::kSfWLoOff, &map_ws, 0, rec_lo + kt * 136 + 128, sfull);
          tma_load_2d(slot + C::kSfWHiOff, &map_ws, 0, rec_hi + kt * 136 + 128, sfull);
          if (!GATHER) tma_load_2d(slot + C::kSfTokOff, &map_sfx, 0, (b * (kH / 128) + 2 * kt) * 4, sfull);
        }
        if (GATHER) {
          __syncwarp();
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            const bool live = soff[m] != 0xffffffffu;
            const uint8_t* src = rows.scales + (live ? soff[m] : 0u) + kt * 8;
            cp_async_4(slot + cell + m * 4, src, live ? 4u : 0u);
            cp_async_4(slot + cell + m * 4 + kAtomBytes, src + 4, live ? 4u : 0u);
          }
          cp_async_arrive(sfull);
        }
      }
    }
    if (GATHER) asm volatile("cp.async.wait_all;" ::: "memory");
    if (!ok && lane == 0) drain_copies(bar_sfull, it, C::kSfStages);
  } else if (GATHER && warp >= C::kGather0 && warp < C::kGather0 + 4) {
    // ---------------------------------------------------------------- token gather: this warp's 32 rows of each block
    const int gw = warp - C::kGather0;
    const int c = lane & 7, sub = lane >> 3;  // 8 lanes x 16 bytes = one 128-byte row slice, 4 rows per instruction
    // rows 32 gw + 4 i + sub: (row & 7) = 4 (i & 1) + sub, so a lane has two destination patterns
    const uint32_t dst_even = static_cast<uint32_t>(C::kTokOff + (32 * gw + sub) * 128 + ((c ^ sub) << 4));
    const uint32_t dst_odd = static_cast<uint32_t>(C::kTokOff + (32 * gw + sub) * 128 + ((c ^ (4 + sub)) << 4));
    const uint8_t* codes = rows.codes + c * 16;
    uint32_t it = 0;
    bool ok = true;
    int ahead = first < total ? __ldcg(sorted_ids + (b_lo + first / C::kTilePairs) * 128 + 32 * gw + lane) : -1;
    for (int u = first; u < total && ok; u += stride) {
      const uint32_t mine = gather_row(ahead, rows);  // the input row of block row 32 gw + lane, ~0: padding
      if (u + stride < total) ahead = __ldcg(sorted_ids + (b_lo + (u + stride) / C::kTilePairs) * 128 + 32 * gw + lane);
      uint32_t off[8];  // byte offset of the row's codes (the host keeps tokens * H/2 below 2^32), ~0: padding
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t t = __shfl_sync(0xffffffffu, mine, 4 * i + sub);
        off[i] = t != 0xffffffffu ? t * static_cast<uint32_t>(kH / 2) : 0xffffffffu;
      }
      for (int kt = 0; kt < kK1Tiles; ++kt, ++it) {
        const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_v, status))) { ok = false; break; }
        const uint32_t base = tiles + s * C::kStageBytes;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const bool live = off[i] != 0xffffffffu;
          cp_async_16(base + i * 512 + ((i & 1) ? dst_odd : dst_even), codes + (live ? off[i] : 0u) + kt * 128,
                      live ? 16u : 0u);
        }
        cp_async_arrive(smem_u32(&bar_full[s]));
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      // E2M1 x E2M1, UE8M0 scales, M = 128 token rows, N = 256 weight rows
      constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(256 >> 3) << 17) | (1u << 23) |
                                  (static_cast<uint32_t>(128 >> 4) << 24);
      constexpr uint32_t kId0 = kIdesc, kId1 = kIdesc | (2u << 29) | (2u << 4);
      uint32_t it = 0, ui = 0;
      bool ok = true;
      for (int u = first; u < total && ok; u += stride, ++ui) {
        if (!mbar_wait(smem_u32(&bar_tempty), (ui & 1u) ^ 1u, abort_v, status)) break;
        tc_fence_after();
        for (int kt = 0; kt < kK1Tiles; ++kt, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          const uint32_t j = it % C::kSfStages, sph = (it / C::kSfStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_sf[j]), sph, abort_v, status)) { ok = false; break; }   // long since complete
          if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_v, status)) { ok = false; break; }  // the wait that matters
          tc_fence_after();
          if (GATHER) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // rows written by plain copies
          const uint32_t lo = (tiles + s * C::kStageBytes) >> 4;
          const uint32_t x_lo = lo + (C::kTokOff >> 4), w_lo = lo + (C::kWOff >> 4);
          const uint32_t t_sft = tmem_base + C::kSfCol + 24u * j, t_sfw = t_sft + 8u;
          tc_mma_mxf4_wide(tmem_base, x_lo, w_lo, kId0, t_sft, t_sfw, static_cast<uint32_t>(kt != 0));
          tc_mma_mxf4_wide(tmem_base, x_lo + 2, w_lo + 2, kId1, t_sft, t_sfw, 1u);
          tc_mma_mxf4_wide(tmem_base, x_lo + 4, w_lo + 4, kId0, t_sft + 4, t_sfw + 8, 1u);
          tc_mma_mxf4_wide(tmem_base, x_lo + 6, w_lo + 6, kId1, t_sft + 4, t_sfw + 8, 1u);
          tc_commit(smem_u32(&bar_empty[s]));
        }
        if (ok) tc_commit(smem_u32(&bar_tfull));
      }
      if (*abort_v) drain_tcgen05(smem_u32(&bar_drain[0]));
    }
  } else if (warp == 2 || warp == 3) {
    // ---------------------------------------------------------------- scale copies (three of the six atoms each)
    if (lane == 0) {
      const bool head = warp == 2;
      uint32_t it = 0;
      bool ok = true;
      for (int u = first; u < total && ok; u += stride) {
        for (int kt = 0; kt < kK1Tiles; ++kt, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          const uint32_t j = it % C::kSfStages, sph = (it / C::kSfStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_sfull[j]), sph, abort_v, status)) { ok = false; break; }
          // scale set j was last read by the MMAs of K-tile it - 8: complete once those of K-tile it - 4 are
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_v, status)) { ok = false; break; }
          tc_fence_after();
          if (GATHER) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          const uint32_t lo = (sf_ring + j * C::kSfSlotBytes) >> 4;
          const uint32_t t_sft = tmem_base + C::kSfCol + 24u * j, t_sfw = t_sft + 8u;
          if (head) {
            tc_cp_scales_lo(t_sft, lo + (C::kSfTokOff >> 4));
            tc_cp_scales_lo(t_sft + 4, lo + ((C::kSfTokOff + kAtomBytes) >> 4));
            tc_cp_scales_lo(t_sfw, lo + (C::kSfWLoOff >> 4));
          } else {
            tc_cp_scales_lo(t_sfw + 4, lo + (C::kSfWHiOff >> 4));
            tc_cp_scales_lo(t_sfw + 8, lo + ((C::kSfWLoOff + kAtomBytes) >> 4));
            tc_cp_scales_lo(t_sfw + 12, lo + ((C::kSfWHiOff + kAtomBytes) >> 4));
          }
          tc_commit(smem_u32(&bar_sf[j]));
        }
      }
      if (*abort_v) drain_tcgen05(smem_u32(&bar_drain[1]));
    }
  }
  } else {
    // ---------------------------------------------------------------- epilogue (eight warps)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
    const int q = warp & 3;
    const int half = ((warp - C::kEpilogue0) >> 2) & 1;
    const int tr = q * 32 + lane;
    uint32_t ui = 0;
    for (int u = first; u < total; u += stride, ++ui) {
      const int b = b_lo + u / C::kTilePairs, tp = u % C::kTilePairs;
      const int64_t row = static_cast<int64_t>(b) * 128 + tr;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_tfull), ui & 1u, abort_v, status))) break;
      tc_fence_after();
      const uint32_t t_acc = tmem_base + 128u * half + (static_cast<uint32_t>(q * 32) << 16);
      uint32_t acc[4][32];
      tc_ld32_nowait(t_acc, acc[0]);
      tc_ld32_nowait(t_acc + 32, acc[1]);
      tc_ld32_nowait(t_acc + 64, acc[2]);
      tc_ld32_nowait(t_acc + 96, acc[3]);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      tc_fence_before();  // the accumulator sits in registers: hand it back, the next unit's MMAs run under the arithmetic
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_tempty));
#pragma unroll
      for (int g = 0; g < 2; ++g)
        swiglu_quant_store(acc[2 * g], acc[2 * g + 1], hq, sfh, row, b, tr, 4 * tp + 2 * half + g);
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

// ------------------------------------------------------------------------------------------------ host side
// byte matrix [rows][128], boxes of 128 bytes x box_rows, no swizzle (the bytes are stored as shared memory wants them)
static int make_flat_map(CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return B200MOE_E_DRIVER;
  const cuuint64_t dims[2] = {128, rows};
  const cuuint64_t strides[1] = {128};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : B200MOE_E_DRIVER;
}

// CTA pairs that can be resident at once on the current device (0: cluster launch unavailable)
static int resident_pairs() {
  static std::mutex mu;
  static int pairs[kMaxDevices] = {};
  static bool known[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (!known[dev]) {
    int n = 0;
    if (cudaFuncSetAttribute(gemm1_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kSmemBytes) ==
        cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * sm_count());
      cfg.blockDim = dim3(PairCfg::kThreads);
      cfg.dynamicSmemBytes = PairCfg::kSmemBytes;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&n, gemm1_pair_kernel, &cfg) != cudaSuccess) n = 0;
    }
    (void)cudaGetLastError();
    pairs[dev] = n;
    known[dev] = true;
  }
  return pairs[dev];
}

int set_wait_limit_pair(unsigned long long ns) { return set_wait_limit_here(ns); }

}  // namespace b200moe

extern "C" int b200moe_gemm1_swiglu_quant_wide(const uint8_t* w13t, int num_experts, const uint8_t* xq_sorted,
                                               const uint8_t* sfx, const int32_t* block_expert, const int32_t* num_valid,
                                               int64_t max_rows, uint8_t* hq, uint8_t* sfh, int32_t* status, void* stream) {
  using namespace b200moe;
  using C = WideCfg;
  if (!w13t || !xq_sorted || !sfx || !block_expert || !num_valid || !hq || !sfh || !status) return B200MOE_E_ARG;
  if (num_experts < 1 || num_experts > kMaxE || max_rows < 0 || max_rows % 128) return B200MOE_E_ARG;
  if (misaligned(w13t, 16) || misaligned(xq_sorted, 16) || misaligned(sfx, 16) || misaligned(hq, 16) || misaligned(sfh, 16))
    return B200MOE_E_ALIGN;
  if (max_rows == 0) return 0;
  CUtensorMap mx, msf, mwc, mws;
  int r = make_map(&mx, xq_sorted, kH / 2, static_cast<uint64_t>(max_rows), 128);
  if (r) return r;
  const uint64_t sf_rows = static_cast<uint64_t>(max_rows / 128) * (kH / 128) * 4;
  if ((r = make_flat_map(&msf, sfx, sf_rows, 8))) return r;
  const uint64_t w_rows = static_cast<uint64_t>(num_experts) * kW13Tiles * kK1Tiles * 136;
  if ((r = make_flat_map(&mwc, w13t, w_rows, 128))) return r;
  if ((r = make_flat_map(&mws, w13t, w_rows, 8))) return r;
  static PerDeviceOnce once;
  const int rc = once.run([] {
    return static_cast<int>(cudaFuncSetAttribute(gemm1_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
  });
  if (rc) return rc;
  const int64_t max_units = max_rows / 128 * C::kTilePairs;
  const int grid = static_cast<int>(max_units < sm_count() ? max_units : sm_count());
  B200MOE_LAUNCH(gemm1_wide_kernel<false>, grid, C::kThreads, C::kSmemBytes, static_cast<cudaStream_t>(stream), mx, msf, mwc,
                 mws, GatherRows{}, block_expert, num_valid, hq, sfh, status, num_experts, static_cast<int>(max_rows / 128),
                 static_cast<const int32_t*>(nullptr));
  return 0;
}

extern "C" int b200moe_gemm1_swiglu_quant_gather_range(const uint8_t* w13t, int num_experts, const uint8_t* codes,
                                                 const uint8_t* scales, int64_t tokens, int by_pair, const int32_t* sorted_ids,
                                                 const int32_t* block_expert, const int32_t* num_valid, int64_t max_rows,
                                                 uint8_t* hq, uint8_t* sfh, const int32_t* block_range, int max_ctas,
                                                 int32_t* status, void* stream) {
  using namespace b200moe;
  using C = WideCfg;
  if (!w13t || !codes || !scales || !sorted_ids || !block_expert || !num_valid || !hq || !sfh || !status)
    return B200MOE_E_ARG;
  if (num_experts < 1 || num_experts > kMaxE || max_rows < 0 || max_rows % 128) return B200MOE_E_ARG;
  if (tokens < 0 || tokens > (1 << 24) - 1) return B200MOE_E_ARG;  // a sorted entry carries the token in its low 24 bits
  if (misaligned(w13t, 16) || misaligned(codes, 16) || misaligned(scales, 4) || misaligned(sorted_ids, 4) ||
      misaligned(hq, 16) || misaligned(sfh, 16))
    return B200MOE_E_ALIGN;
  if (max_rows == 0) return 0;
  CUtensorMap mwc, mws;
  int r;
  const uint64_t w_rows = static_cast<uint64_t>(num_experts) * kW13Tiles * kK1Tiles * 136;
  if ((r = make_flat_map(&mwc, w13t, w_rows, 128))) return r;
  if ((r = make_flat_map(&mws, w13t, w_rows, 8))) return r;
  static PerDeviceOnce once;
  const int rc = once.run([] {
    return static_cast<int>(cudaFuncSetAttribute(gemm1_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
  });
  if (rc) return rc;
  const int64_t max_units = max_rows / 128 * C::kTilePairs;
  int grid = static_cast<int>(max_units < sm_count() ? max_units : sm_count());
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  const GatherRows rows{codes, scales, sorted_ids, tokens, by_pair ? 1 : 0};
  B200MOE_LAUNCH(gemm1_wide_kernel<true>, grid, C::kThreads, C::kSmemBytes, static_cast<cudaStream_t>(stream), mwc, mwc, mwc,
                 mws, rows, block_expert, num_valid, hq, sfh, status, num_experts, static_cast<int>(max_rows / 128), block_range);
  return 0;
}

extern "C" int b200moe_gemm1_swiglu_quant_gather(const uint8_t* w13t, int num_experts, const uint8_t* codes,
                                                 const uint8_t* scales, int64_t tokens, int by_pair, const int32_t* sorted_ids,
                                                 const int32_t* block_expert, const int32_t* num_valid, int64_t max_rows,
                                                 uint8_t* hq, uint8_t* sfh, int32_t* status, void* stream) {
  return b200moe_gemm1_swiglu_quant_gather_range(w13t, num_experts, codes, scales, tokens, by_pair, sorted_ids, block_expert,
                                                 num_valid, max_rows, hq, sfh, nullptr, 0, status, stream);
}

extern "C" int b200moe_gemm1_pair_supported(void) { return b200moe::resident_pairs() > 0 ? 1 : 0; }

extern "C" int b200moe_gemm1_swiglu_quant_pair(const uint8_t* w13t, int num_experts, const uint8_t* xq_sorted,
                                               const uint8_t* sfx, const int32_t* block_expert, const int32_t* num_valid,
                                               int64_t max_rows, uint8_t* hq, uint8_t* sfh, int32_t* status, void* stream) {
  using namespace b200moe;
  if (!w13t || !xq_sorted || !sfx || !block_expert || !num_valid || !hq || !sfh || !status) return B200MOE_E_ARG;
  if (num_experts < 1 || num_experts > kMaxE || max_rows < 0 || max_rows % 128 || max_rows / 128 > PairCfg::kMaxBlocks)
    return B200MOE_E_ARG;
  if (misaligned(w13t, 16) || misaligned(xq_sorted, 16) || misaligned(sfx, 16) || misaligned(hq, 16) || misaligned(sfh, 16))
    return B200MOE_E_ALIGN;
  if (max_rows == 0) return 0;
  const int pairs = resident_pairs();
  if (pairs <= 0) return B200MOE_E_DRIVER;
  CUtensorMap mx, msf, mwc, mws;
  int r = make_map(&mx, xq_sorted, kH / 2, static_cast<uint64_t>(max_rows), 128);
  if (r) return r;
  const uint64_t sf_rows = static_cast<uint64_t>(max_rows / 128) * (kH / 128) * 4;
  if ((r = make_flat_map(&msf, sfx, sf_rows, 8))) return r;
  const uint64_t w_rows = static_cast<uint64_t>(num_experts) * kW13Tiles * kK1Tiles * 136;
  if ((r = make_flat_map(&mwc, w13t, w_rows, 128))) return r;
  if ((r = make_flat_map(&mws, w13t, w_rows, 8))) return r;
  const int64_t max_units = max_rows / 128 * PairCfg::kTilePairs;
  const int clusters = static_cast<int>(max_units < pairs ? max_units : pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(PairCfg::kThreads);
  cfg.dynamicSmemBytes = PairCfg::kSmemBytes;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm1_pair_kernel, mx, msf, mwc, mws, block_expert, num_valid, hq, sfh,
                                           status, num_experts, static_cast<int>(max_rows / 128));
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
