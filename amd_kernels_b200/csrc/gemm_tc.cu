// Grouped MXFP4 x MXFP4 GEMMs on the sm_100a tensor cores (tcgen05.mma kind::mxf4, block scale per 32, fp32
// accumulators in tensor memory), one persistent CTA per SM.
//
// Orientation: the weight tile is the 128-row M operand, the expert's token block (16/32/64/128 sorted rows) is the N
// operand. So one pass over an expert's weights serves its whole block, the accumulator of output feature i sits in TMEM
// lane i, and a token is a TMEM column.
//
//   warp 0    producer: one thread issues the bulk copies of weight tile records and scale atoms and the TMA tile loads of
//             the token codes
//   warp 1    MMA: allocates TMEM; one thread issues tcgen05.mma, four per stage
//   last warp scale copies: one thread moves each stage's scale atoms into TMEM (tcgen05.cp), stages ahead of the MMAs.
//             Two issuing threads because every tcgen05 / mbarrier instruction costs its thread ~50 cycles whatever the
//             size of the MMA, and one thread doing both was what bounded the kernel
//   (the one-launch kernel gemm12_kernel also has warp 6: a second producer for the token-side operand)
//   warps 2-5 epilogue (bm = 128: a second group, warps 6-9, takes every other unit): tcgen05.ld of the accumulator, then
//             GEMM1: SwiGLU-OAI (gate and up rows of one tile live in neighbouring lane quarters), MXFP4 requantisation
//                    of 32 intermediate columns = the 32 lanes of a warp, codes and scale atoms to global memory
//             GEMM2: times the routing weight, bf16, one store per (token, slot, column)
//
// Every mbarrier wait is bounded: after about two seconds it records B200MOE_DEV_TIMEOUT in the status word, raises a
// CTA-wide abort flag, the roles drain and the CTA frees its TMEM and returns.
#include "tc_host.cuh"
#include "tc_ptx.cuh"

namespace b200moe {

// ------------------------------------------------------------------------------------------------ kernel
template <int MODE, int BM>
struct Cfg {
  static constexpr int kTilesM = MODE == 1 ? kW13Tiles : kW2Tiles;
  static constexpr int kTilesK = MODE == 1 ? kK1Tiles : kK2Tiles;
  static constexpr int kABytes = 128 * 128;
  static constexpr int kSfBytes = 2 * kAtomBytes;
  static constexpr int kBBytes = BM * 128;
  // stage = [weight tile record: codes | scales][activation codes][activation scales]
  static constexpr int kBOffset = kTileRecordBytes;
  static constexpr int kSfbOffset = kBOffset + kBBytes;
  static constexpr int kStageBytes = kSfbOffset + kSfBytes;
  // bm = 128 (prefill): the token block is the 128-row M operand and the weight tile is N, so a TMEM lane is a token and
  // the epilogue works on registers alone. Smaller blocks: the weight tile is M and the tokens are N (any multiple of 16).
  static constexpr bool kTokensAreM = BM == 128;
  static constexpr int kAccBufs = 2;
  static constexpr int kStages = BM == 128 ? (MODE == 1 ? 6 : 5) : (MODE == 1 && BM == 64 ? 6 : 8);
  // bm = 128 GEMM2 runs two epilogue groups of four warps, one per TMEM accumulator buffer, on alternate units
  static constexpr int kEpiGroups = kTokensAreM ? 2 : 1;
  // warps: 0 = copy producer, 1 = MMA issue, 2 .. = epilogue groups, last = scale-copy issue
  static constexpr int kThreads = 64 + 128 * kEpiGroups + 32;
  static constexpr int kScaleWarp = 2 + 4 * kEpiGroups;
  static constexpr int kAccCols = BM;  // fp32 accumulator columns per buffer
  // scale columns behind the accumulators: kSfSets sets of (8 for the weight tile + 8 for the token tile), used in
  // rotation: the scale copies are issued by their own thread, stages ahead of the MMAs that read them
  static constexpr int kSfSets = 8;  // >= kStages: a set is reused only after its MMAs completed
  static_assert(kSfSets >= kStages, "scale sets");
  static constexpr int kSfaCol = kAccBufs * kAccCols;
  static constexpr int kSfbCol = kSfaCol + 8;
  static constexpr int kColsUsed = kSfaCol + 16 * kSfSets;
  static constexpr int kTmemCols = kColsUsed <= 64 ? 64 : (kColsUsed <= 128 ? 128 : (kColsUsed <= 256 ? 256 : 512));
  // GEMM1 epilogue staging: up to 64 token columns x (2 groups x (32 gate + 32 up + 4 pad)) floats
  static constexpr int kEpiCols = BM < 64 ? BM : 64;
  static constexpr int kEpiRowFloats = 136;
  // GEMM2 epilogue staging: up to 32 token columns x (128 output columns + 4 pad) floats
  static constexpr int kOutCols = BM < 32 ? BM : 32;
  static constexpr int kOutRowFloats = 132;
  // bm = 128 GEMM2: one strip of 32 rows x (128 bytes + 16 pad) per epilogue warp
  static constexpr int kStripRowBytes = 144;
  static constexpr int kEpiBytes = kTokensAreM ? (MODE == 2 ? 8 * 32 * kStripRowBytes : 0)
                                               : (MODE == 1 ? kEpiCols * kEpiRowFloats * 4 : kOutCols * kOutRowFloats * 4);
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024;  // + slack to align to 1024 bytes
  static constexpr int kActAtomsPerBlock = MODE == 1 ? kH / 128 : kI / 128;  // activation scale atoms per row block
  static constexpr int kActRowBytes = MODE == 1 ? kH / 2 : kI / 2;
};

struct EpilogueArgs {
  // GEMM1
  uint8_t* hq;
  uint8_t* sfh;
  const uint8_t* next_tiles;  // GEMM1, may be null: the W2 tile records, prefetched into L2 for the GEMM2 that follows
  // GEMM2
  const int32_t* sorted_ids;
  const float* sorted_w;
  __nv_bfloat16* slots;
  int64_t tokens;
  // GEMM2, expert parallel: pair r of this rank's rows belongs to rank row_rank[r], where it is pair row_pair[r];
  // its result row is stored straight into that rank's slot buffer peer_slots[rank] (a peer mapping over NVLink)
  const int32_t* row_rank;
  const int32_t* row_pair;
  __nv_bfloat16* peer_slots[8];
  int world;
  int64_t peer_rows;  // rows of every rank's slot buffer
  int32_t* status;
  // may be null; otherwise the launch covers the row blocks [block_range[0], block_range[1]) only (a caller that splits the
  // row blocks into chunks, so that this kernel can start on one chunk while its predecessor works on the next)
  const int32_t* block_range;
  int max_ctas;  // host side only: > 0 caps the grid (leaves SMs to a kernel that runs beside this one)
};

// What the GEMM2 epilogue needs to place a result row, held in registers / shared memory (never indexed dynamically
// inside the kernel-parameter struct, which would push the whole struct into local memory).
struct RowPlacer {
  __nv_bfloat16* slots;
  int64_t tokens;
  const int32_t* row_rank;
  const int32_t* row_pair;
  __nv_bfloat16* const* peers;  // shared-memory copy of the peer table
  int world;
  int64_t peer_rows;
  int32_t* status;
  // Where the result row of sorted-row entry `sid` goes (null: a padding row).
  __device__ __forceinline__ __nv_bfloat16* row(int sid) const {
    const int64_t token = sid & 0x00ffffff;
    if (token >= tokens) return nullptr;
    const int64_t pair = token * kTopK + ((sid >> 24) & 3);
    if (row_rank == nullptr) return slots + pair * kH;
    const int rank = __ldcg(row_rank + pair);
    const int64_t dst_pair = __ldcg(row_pair + pair);
    if (rank < 0 || rank >= world || dst_pair < 0 || dst_pair >= peer_rows) {  // never store through a bad index
      atomicExch(status, B200MOE_DEV_BAD_INDEX);
      return nullptr;
    }
    return peers[rank] + dst_pair * kH;
  }
};

// Copies the fields of the kernel parameter into registers (laundered: they point at data a predecessor kernel wrote)
// and the peer table into shared memory. Call after pdl_wait(), before the roles split; `s_peer` is a __shared__ array.
__device__ __forceinline__ RowPlacer make_placer(const EpilogueArgs& ep, __nv_bfloat16** s_peer) {
  if (threadIdx.x == 0) {
#pragma unroll
    for (int r = 0; r < 8; ++r) s_peer[r] = ep.peer_slots[r];
  }
  RowPlacer p;
  p.slots = ep.slots;
  p.tokens = ep.tokens;
  p.row_rank = ep.row_rank;
  p.row_pair = ep.row_pair;
  p.peers = s_peer;
  p.world = ep.world;
  p.peer_rows = ep.peer_rows;
  p.status = ep.status;
  launder(p.row_rank);
  launder(p.row_pair);
  return p;
}

template <int MODE, int BM>
__global__ void __launch_bounds__((Cfg<MODE, BM>::kThreads), 1)
    grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const uint8_t* __restrict__ w_tiles,
                        const uint8_t* __restrict__ sf_x, const int32_t* __restrict__ block_expert,
                        const int32_t* __restrict__ num_valid, EpilogueArgs ep, int32_t* status, int num_experts,
                        int max_blocks) {
  using C = Cfg<MODE, BM>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[C::kStages];
  __shared__ __align__(8) uint64_t bar_empty[C::kStages];
  __shared__ __align__(8) uint64_t bar_sf[C::kStages];  // the stage's scales are in tensor memory
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ __align__(8) uint64_t bar_drain[2];  // used after an abort only
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ __nv_bfloat16* s_dst[MODE == 2 ? BM : 1];
  __shared__ __nv_bfloat16* s_peer[8];
  __shared__ float s_wt[MODE == 2 ? BM : 1];

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

  // barriers and TMEM are set up; from here on the kernel reads what its predecessors wrote
  pdl_wait();
  launder(w_tiles);
  launder(sf_x);
  launder(block_expert);
  launder(num_valid);
  const int32_t* sorted_ids = ep.sorted_ids;
  const float* sorted_w = ep.sorted_w;
  launder(sorted_ids);
  launder(sorted_w);
  const RowPlacer placer = make_placer(ep, s_peer);
  __syncthreads();
  int n_blocks = __ldcg(num_valid) / BM;
  if (n_blocks < 0 || n_blocks > max_blocks) {  // a routing table that does not fit its buffers: record it, do nothing
    if (threadIdx.x == 0) atomicExch(status, B200MOE_DEV_BAD_INDEX);
    n_blocks = 0;
  }
  int b_lo = 0;
  if (ep.block_range != nullptr) {
    const int32_t* range = ep.block_range;
    launder(range);
    b_lo = max(0, min(__ldcg(range), n_blocks));
    n_blocks = max(b_lo, min(__ldcg(range + 1), n_blocks)) - b_lo;
  }
  const int total_units = n_blocks * C::kTilesM;

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      bool ok = true;
      // slot state kept incrementally (no division in the loop): shared-memory address, barriers, phase
      const uint32_t full0 = smem_u32(&bar_full[0]), empty0 = smem_u32(&bar_empty[0]);
      uint32_t it = 0, slot = 0, ph = 1u, base = tiles, full = full0, empty = empty0;
      // the expert id of a unit is fetched one unit ahead: a GEMM2 unit is only three stages long, and an L2 round trip
      // in front of each would leave the copy queue short
      int e_ahead = static_cast<int>(blockIdx.x) < total_units ? __ldcg(block_expert + b_lo + blockIdx.x / C::kTilesM) : 0;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        const int b = b_lo + u / C::kTilesM, mt = u % C::kTilesM;
        int e = e_ahead;
        const int un = u + static_cast<int>(gridDim.x);
        if (un < total_units) e_ahead = __ldcg(block_expert + b_lo + un / C::kTilesM);
        if (e < 0 || e >= num_experts) {  // never form an address from an expert id outside the weights
          atomicExch(status, B200MOE_DEV_BAD_INDEX);
          e = 0;
        }
        const uint8_t* w_src = w_tiles + static_cast<int64_t>(e * C::kTilesM + mt) * C::kTilesK * kTileRecordBytes;
        const uint8_t* sfb_src = sf_x + static_cast<int64_t>(b) * C::kActAtomsPerBlock * kAtomBytes;
        const int row0 = b * BM;
        for (int kt = 0; kt < C::kTilesK; ++kt, ++it) {
          if (!mbar_wait(empty, ph, abort_v, status)) { ok = false; break; }
          mbar_arrive_expect_tx(full, C::kStageBytes);
          bulk_load(base, w_src, kTileRecordBytes, full);
          tma_load_2d(base + C::kBOffset, &map_x, kt * 128, row0, full);
          bulk_load(base + C::kSfbOffset, sfb_src, C::kSfBytes, full);
          w_src += kTileRecordBytes;
          sfb_src += C::kSfBytes;
          if (++slot == C::kStages) {
            slot = 0; ph ^= 1u; base = tiles; full = full0; empty = empty0;
          } else {
            base += C::kStageBytes; full += 8; empty += 8;
          }
        }
      }
      if (MODE == 1 && ok && ep.next_tiles != nullptr) {
        // This CTA's weight stream has ended: ask L2 for the W2 tiles that the following GEMM2 reads first (its unit u2 =
        // row block u2 / 48, tile u2 % 48; four rounds of one unit per SM), while the slower CTAs finish.
        const int lim = total_units / C::kTilesM * kW2Tiles < 592 ? total_units / C::kTilesM * kW2Tiles : 592;
        for (int u2 = blockIdx.x; u2 < lim; u2 += gridDim.x) {
          const int e = __ldcg(block_expert + u2 / kW2Tiles);
          if (e >= 0 && e < num_experts)
            l2_prefetch_bulk(ep.next_tiles + static_cast<int64_t>(e * kW2Tiles + u2 % kW2Tiles) * kK2Tiles * kTileRecordBytes,
                             kK2Tiles * kTileRecordBytes);
        }
      }
      if (!ok) {
        // aborting: let the copies already in flight land before the CTA gives up its shared memory
        drain_copies(bar_full, it, C::kStages);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BM >> 3) << 17) | (1u << 23) | (8u << 24);
      // The instruction stream of one thread bounds this kernel (every tcgen05 / mbarrier instruction costs it ~50
      // cycles), so the per-stage work is split: the scale-copy thread (last warp) waits for the stage's bytes and copies
      // its scales into tensor memory; this thread waits for that and issues the four MMAs. State is kept incrementally:
      // the slot's shared-memory address >> 4 (the low word of every descriptor), its barriers, the phase, the scale set.
      const uint32_t sf0 = smem_u32(&bar_sf[0]), empty0 = smem_u32(&bar_empty[0]);
      uint32_t slot = 0, ph = 0, sfset = 0, ui = 0;
      uint32_t lo = tiles >> 4, full = sf0, empty = empty0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++ui) {
        const uint32_t acc = ui & 1u, aph = (ui >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tempty[acc]), aph ^ 1u, abort_v, status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::kAccCols;
        for (int kt = 0; kt < C::kTilesK; ++kt) {
          if (!mbar_wait(full, ph, abort_v, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t t_sfa = tmem_base + C::kSfaCol + 16u * sfset, t_sfb = t_sfa + 8u;
          // 64 elements = 32 bytes (descriptor + 2) per MMA; scales: atom k/2, bytes {0,1} or {2,3} of each row's cell
          constexpr uint32_t kId0 = kIdesc, kId1 = kIdesc | (2u << 29) | (2u << 4);
          const uint32_t w_lo = lo, x_lo = lo + (C::kBOffset >> 4);
          if (C::kTokensAreM) {
            tc_mma_mxf4_lo<2>(d_tmem, x_lo, w_lo, kId0, t_sfb, t_sfa, static_cast<uint32_t>(kt != 0));
            tc_mma_mxf4_lo<1>(d_tmem, x_lo + 2, w_lo + 2, kId1, t_sfb, t_sfa);
            tc_mma_mxf4_lo<1>(d_tmem, x_lo + 4, w_lo + 4, kId0, t_sfb + 4, t_sfa + 4);
            tc_mma_mxf4_lo<1>(d_tmem, x_lo + 6, w_lo + 6, kId1, t_sfb + 4, t_sfa + 4);
          } else {
            tc_mma_mxf4_lo<2>(d_tmem, w_lo, x_lo, kId0, t_sfa, t_sfb, static_cast<uint32_t>(kt != 0));
            tc_mma_mxf4_lo<1>(d_tmem, w_lo + 2, x_lo + 2, kId1, t_sfa, t_sfb);
            tc_mma_mxf4_lo<1>(d_tmem, w_lo + 4, x_lo + 4, kId0, t_sfa + 4, t_sfb + 4);
            tc_mma_mxf4_lo<1>(d_tmem, w_lo + 6, x_lo + 6, kId1, t_sfa + 4, t_sfb + 4);
          }
          tc_commit(empty);
          sfset = (sfset + 1u) & (C::kSfSets - 1);
          if (++slot == C::kStages) {
            slot = 0; ph ^= 1u; lo = tiles >> 4; full = sf0; empty = empty0;
          } else {
            lo += C::kStageBytes >> 4; full += 8; empty += 8;
          }
        }
        if (ok) tc_commit(smem_u32(&bar_tfull[acc]));
      }
      if (*abort_v) drain_tcgen05(smem_u32(&bar_drain[0]));
    }
  } else if (warp == C::kScaleWarp) {
    // ---------------------------------------------------------------- scale copies: shared memory -> tensor memory
    if (lane == 0) {
      const uint32_t full0 = smem_u32(&bar_full[0]), sf0 = smem_u32(&bar_sf[0]);
      uint32_t slot = 0, ph = 0, sfset = 0;
      uint32_t lo = tiles >> 4, full = full0, sf = sf0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        for (int kt = 0; kt < C::kTilesK; ++kt) {
          // full: the stage's bytes have landed, and (through the producer's wait) the MMAs that last read this slot and
          // this scale set, kStages <= kSfSets stages ago, have completed
          if (!mbar_wait(full, ph, abort_v, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t t_sfa = tmem_base + C::kSfaCol + 16u * sfset, t_sfb = t_sfa + 8u;
          tc_cp_scales_lo(t_sfa, lo + (C::kABytes >> 4));
          tc_cp_scales_lo(t_sfa + 4, lo + ((C::kABytes + kAtomBytes) >> 4));
          tc_cp_scales_lo(t_sfb, lo + (C::kSfbOffset >> 4));
          tc_cp_scales_lo(t_sfb + 4, lo + ((C::kSfbOffset + kAtomBytes) >> 4));
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
    // ---------------------------------------------------------------- epilogue (groups of 4 warps, TMEM lane quarter = warp % 4)
    const int q = warp & 3;
    const int group = (warp - 2) >> 2;                   // epilogue group 0 or 1
    const int et = (threadIdx.x - 64) & 127;             // 0..127, work-item index inside the group
    const int tr = q * 32 + lane;     // the TMEM lane this thread reads (warps 2..5 own quarters 2, 3, 0, 1)
    float* stage_f = reinterpret_cast<float*>(smem_raw + (tiles - smem_u32(smem_raw)) + C::kStages * C::kStageBytes);
    uint32_t ui = 0;
    bool have_ahead = false;
    int ahead_sid = 0;
    float ahead_wt = 0.0f;
    for (int u = blockIdx.x; u < total_units; u += gridDim.x, ++ui) {
      if (C::kEpiGroups == 2 && static_cast<int>(ui & 1u) != group) continue;  // group g owns accumulator buffer g
      const int b = b_lo + u / C::kTilesM, mt = u % C::kTilesM;
      const uint32_t acc = ui & 1u, aph = (ui >> 1) & 1u;
      const int64_t row0 = static_cast<int64_t>(b) * BM;
      __nv_bfloat16* my_dst = nullptr;
      float my_wt = 0.0f;
      if (MODE == 2 && C::kTokensAreM) {  // one token row per thread; fetched before the wait, hidden behind the MMAs
        my_dst = placer.row(__ldcg(sorted_ids + row0 + tr));
        my_wt = __ldcg(sorted_w + row0 + tr);
      } else if (MODE == 2 && et < BM) {
        // this block's rows; normally fetched one unit ahead (below), so no memory round trip sits in front of the wait
        if (!have_ahead) {
          ahead_sid = __ldcg(sorted_ids + row0 + et);
          ahead_wt = __ldcg(sorted_w + row0 + et);
        }
        s_dst[et] = placer.row(ahead_sid);
        s_wt[et] = ahead_wt;
      }
      // the four warps must agree before they meet at the named barrier below
      if (!epilogue_all(mbar_wait(smem_u32(&bar_tfull[acc]), aph, abort_v, status), 1u + group)) break;
      tc_fence_after();
      if (MODE == 2 && !C::kTokensAreM) {  // look ahead: the rows of this CTA's next unit
        const int un = u + static_cast<int>(gridDim.x);
        have_ahead = un < total_units;
        if (have_ahead && et < BM) {
          const int64_t r1 = static_cast<int64_t>(b_lo + un / C::kTilesM) * BM + et;
          ahead_sid = __ldcg(sorted_ids + r1);
          ahead_wt = __ldcg(sorted_w + r1);
        }
      }
      const uint32_t t_acc = tmem_base + acc * C::kAccCols + (static_cast<uint32_t>(q * 32) << 16);
      if (C::kTokensAreM && MODE == 1) {
        // lane = token row tr of the block; columns = tile rows: [gate 32 | up 32 | gate 32 | up 32] of 64 intermediate
        // columns. Everything is thread-local: SwiGLU, the two block maxima, 2 x 32 codes -> two 16-byte stores.
#pragma unroll 1
        for (int g = 0; g < 2; ++g) {
          uint32_t gv[32], uv[32];
          tc_ld32(t_acc + 64 * g, gv);
          tc_ld32(t_acc + 64 * g + 32, uv);
          if (g == 1) {  // accumulator fully read: hand the TMEM buffer back to the MMA warp
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_tempty[acc]));
          }
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
            for (int k = 0; k < 4; ++k)
              acc_w |= cvt_e2m1x2(h[8 * wd + 2 * k] * inv, h[8 * wd + 2 * k + 1] * inv) << (8 * k);
            words[wd] = acc_w;
          }
          const int grp = 2 * mt + g;
          *reinterpret_cast<uint4*>(ep.hq + (row0 + tr) * (kI / 2) + grp * 16) =
              make_uint4(words[0], words[1], words[2], words[3]);
          ep.sfh[(static_cast<int64_t>(b) * (kI / 128) + (grp >> 2)) * kAtomBytes + atom_offset(tr, grp & 3)] =
              static_cast<uint8_t>(sc);
        }
      } else if (C::kTokensAreM) {
        // lane = token row tr; columns = 128 output columns of this W2 tile. Scale, round to bf16, then pass the warp's
        // 32 rows through its own shared-memory strip so that eight lanes store one row's 128 contiguous bytes: full
        // lines for local HBM and full-size packets when the row lives in another rank's slot buffer over NVLink.
        uint8_t* strip = reinterpret_cast<uint8_t*>(stage_f) + (warp - 2) * (32 * C::kStripRowBytes);
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t v[32];
            tc_ld32(t_acc + 64 * half + 32 * c, v);
            if (half == 1 && c == 1) {
              tc_fence_before();
              mbar_arrive(smem_u32(&bar_tempty[acc]));
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              uint32_t o[4];
#pragma unroll
              for (int jj = 0; jj < 4; ++jj) {
                const __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(v[8 * k + 2 * jj]) * my_wt,
                                                                __uint_as_float(v[8 * k + 2 * jj + 1]) * my_wt);
                o[jj] = *reinterpret_cast<const uint32_t*>(&p2);
              }
              *reinterpret_cast<uint4*>(strip + lane * C::kStripRowBytes + c * 64 + k * 16) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3);
            const unsigned long long p =
                __shfl_sync(0xffffffffu, static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(my_dst)), r);
            const uint4 val = *reinterpret_cast<const uint4*>(strip + r * C::kStripRowBytes + (lane & 7) * 16);
            if (p != 0ull)
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(static_cast<uintptr_t>(p)) + mt * 128 + half * 64 +
                                        (lane & 7) * 8) = val;
          }
          __syncwarp();
        }
      } else if (MODE == 1) {
        // TMEM lanes of a tile: quarter 0 = gate i 0..31, 1 = up i 0..31, 2 = gate i 32..63, 3 = up i 32..63.
        // Stage the accumulators as [token][group][32 gate | 32 up | pad] so one thread owns one (token, 32-column
        // group): SwiGLU, the block maximum and the 32 codes are thread-local and the codes leave as one 16-byte store.
        float* mine = stage_f + (q >> 1) * 68 + (q & 1) * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BM; c0 += C::kEpiCols) {
#pragma unroll 1
          for (int cc = 0; cc < C::kEpiCols; cc += 16) {
            uint32_t v[16];
            tc_ld16(t_acc + c0 + cc, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) mine[(cc + j) * C::kEpiRowFloats] = __uint_as_float(v[j]);
          }
          if (c0 + C::kEpiCols >= BM) {  // accumulator fully read: hand the TMEM buffer back to the MMA warp
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_tempty[acc]));
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          for (int item = et; item < 2 * C::kEpiCols; item += 128) {
            const int j = item >> 1, g = item & 1;
            const float4* src = reinterpret_cast<const float4*>(stage_f + j * C::kEpiRowFloats + g * 68);
            float h[32];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float4 gv = src[k], uv = src[8 + k];
              h[4 * k + 0] = swiglu_oai(gv.x, uv.x);
              h[4 * k + 1] = swiglu_oai(gv.y, uv.y);
              h[4 * k + 2] = swiglu_oai(gv.z, uv.z);
              h[4 * k + 3] = swiglu_oai(gv.w, uv.w);
            }
            float amax = 0.0f;
#pragma unroll
            for (int k = 0; k < 32; ++k) amax = fmaxf(amax, fabsf(h[k]));
            const int sc = quark_even_e8m0(amax);
            const float inv = __uint_as_float(static_cast<uint32_t>(254 - sc) << 23);
            uint32_t words[4];
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
              uint32_t acc_w = 0;
#pragma unroll
              for (int k = 0; k < 4; ++k)
                acc_w |= cvt_e2m1x2(h[8 * wd + 2 * k] * inv, h[8 * wd + 2 * k + 1] * inv) << (8 * k);
              words[wd] = acc_w;
            }
            const int grp = 2 * mt + g;  // 32-column group of the intermediate, 0..23
            const int n = c0 + j;
            *reinterpret_cast<uint4*>(ep.hq + (row0 + n) * (kI / 2) + grp * 16) =
                make_uint4(words[0], words[1], words[2], words[3]);
            ep.sfh[(static_cast<int64_t>(b) * (kI / 128) + (grp >> 2)) * kAtomBytes + atom_offset(n, grp & 3)] =
                static_cast<uint8_t>(sc);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      } else {
        // Stage the accumulators as [token][128 columns] so a warp writes one token's 128 columns as 256 contiguous bytes.
        float* mine = stage_f + q * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BM; c0 += C::kOutCols) {
#pragma unroll
          for (int cc = 0; cc < C::kOutCols; cc += 16) {
            uint32_t v[16];
            tc_ld16(t_acc + c0 + cc, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) mine[(cc + j) * C::kOutRowFloats] = __uint_as_float(v[j]);
          }
          if (c0 + C::kOutCols >= BM) {
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_tempty[acc]));
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll 2
          for (int item = et; item < C::kOutCols * 32; item += 128) {
            const int j = item >> 5, seg = item & 31;
            __nv_bfloat16* row_dst = s_dst[c0 + j];
            if (row_dst != nullptr) {
              const float s_w = s_wt[c0 + j];
              const float4 v = *reinterpret_cast<const float4*>(stage_f + j * C::kOutRowFloats + seg * 4);
              const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * s_w, v.y * s_w);
              const __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * s_w, v.w * s_w);
              uint2 packed;
              packed.x = *reinterpret_cast<const uint32_t*>(&lo);
              packed.y = *reinterpret_cast<const uint32_t*>(&hi);
              *reinterpret_cast<uint2*>(row_dst + mt * 128 + seg * 4) = packed;
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
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

// ------------------------------------------------------------------------------------------------ GEMM1 + GEMM2 in one launch
// Decode sizes (bm < 128): both grouped GEMMs as ONE persistent kernel. The unit list is all GEMM1 units followed by all
// GEMM2 units, dealt round-robin to the CTAs, so every CTA finishes its GEMM1 units before its first GEMM2 unit. A GEMM2
// unit of row block b needs the 12 GEMM1 tiles of b: each GEMM1 epilogue publishes its stores (fence, then one atomic
// add on done[b]) and the GEMM2 producer waits -- bounded like every other wait -- until done[b] == 12 before it loads h.
// GEMM1 units never wait, so progress does not depend on scheduling order. What this buys over two launches: no ramp
// between the kernels, and the short GEMM2 units (52 KB of weights) fill the uneven last round of GEMM1 (418 KB units).
template <int BM>
struct Cfg12 {
  using C1 = Cfg<1, BM>;
  static constexpr int kStageBytes = C1::kStageBytes;
  static constexpr int kStages = BM == 64 ? 6 : 8;
  static constexpr int kEpi1 = Cfg<1, BM>::kEpiBytes, kEpi2 = Cfg<2, BM>::kEpiBytes;
  static constexpr int kEpiBytes = kEpi1 > kEpi2 ? kEpi1 : kEpi2;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024;
};

__device__ __forceinline__ bool wait_count(const int32_t* counter, int target, volatile int* abort_flag, int32_t* status) {
  const uint64_t t0 = global_timer();
  uint32_t spins = 0;
  while (true) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    if (v >= target) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer() - t0 > wait_limit_ns()) {
        *abort_flag = 1;
        atomicExch(status, B200MOE_DEV_TIMEOUT);
        return false;
      }
    }
  }
}

template <int BM>
__global__ void __launch_bounds__(256, 1)
    gemm12_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_h,
                  const uint8_t* __restrict__ w13t, const uint8_t* __restrict__ w2t, const uint8_t* __restrict__ sf_x,
                  const int32_t* __restrict__ block_expert, const int32_t* __restrict__ num_valid, EpilogueArgs ep,
                  int32_t* done, int32_t* status, int num_experts, int max_blocks) {
  using C = Cfg<1, BM>;  // stage layout, TMEM columns and epilogue geometry are those of the swap orientation
  using C2 = Cfg<2, BM>;
  using CC = Cfg12<BM>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[CC::kStages];
  __shared__ __align__(8) uint64_t bar_empty[CC::kStages];
  __shared__ __align__(8) uint64_t bar_sf[CC::kStages];  // the stage's scales are in tensor memory (warp 7 copies them)
  __shared__ __align__(8) uint64_t bar_tfull[2];
  __shared__ __align__(8) uint64_t bar_tempty[2];
  __shared__ __align__(8) uint64_t bar_drain[2];  // used after an abort only
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ __nv_bfloat16* s_dst[BM];
  __shared__ __nv_bfloat16* s_peer[8];
  __shared__ float s_wt[BM];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile int* abort_v = &abort_flag;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < CC::kStages; ++s) {
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
  launder(w13t);
  launder(w2t);
  launder(sf_x);
  launder(block_expert);
  launder(num_valid);
  const int32_t* sorted_ids = ep.sorted_ids;
  const float* sorted_w = ep.sorted_w;
  launder(sorted_ids);
  launder(sorted_w);
  const RowPlacer placer = make_placer(ep, s_peer);
  __syncthreads();
  int n_blocks = __ldcg(num_valid) / BM;
  if (n_blocks < 0 || n_blocks > max_blocks) {
    if (threadIdx.x == 0) atomicExch(status, B200MOE_DEV_BAD_INDEX);
    n_blocks = 0;
  }
  const int units1 = n_blocks * kW13Tiles;
  const int total_units = units1 + n_blocks * kW2Tiles;

  if (warp == 0) {
    // ---------------------------------------------------------------- weight producer: arms each stage, streams tile records
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      auto block_of = [&](int u) { return u >= units1 ? (u - units1) / kW2Tiles : u / kW13Tiles; };
      // the expert id of a unit is fetched one unit ahead (a GEMM2 unit is only three stages long)
      int e_ahead = static_cast<int>(blockIdx.x) < total_units ? __ldcg(block_expert + block_of(blockIdx.x)) : 0;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        const bool second = u >= units1;
        const int v = second ? u - units1 : u;
        const int tiles_m = second ? kW2Tiles : kW13Tiles, tiles_k = second ? kK2Tiles : kK1Tiles;
        const int mt = v % tiles_m;
        int e = e_ahead;
        const int un = u + static_cast<int>(gridDim.x);
        if (un < total_units) e_ahead = __ldcg(block_expert + block_of(un));
        if (e < 0 || e >= num_experts) {
          atomicExch(status, B200MOE_DEV_BAD_INDEX);
          e = 0;
        }
        const uint8_t* w_src = (second ? w2t : w13t) + static_cast<int64_t>(e * tiles_m + mt) * tiles_k * kTileRecordBytes;
        for (int kt = 0; kt < tiles_k; ++kt, ++it) {
          const uint32_t s = it % CC::kStages, ph = (it / CC::kStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_v, status)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[s]);
          mbar_arrive_expect_tx(full, C::kStageBytes);  // the whole stage: the activation producer's bytes included
          bulk_load(tiles + s * C::kStageBytes, w_src + static_cast<int64_t>(kt) * kTileRecordBytes, kTileRecordBytes, full);
        }
      }
      if (!ok) {
        drain_copies(bar_full, it, CC::kStages);
      }
    }
  } else if (warp == 6) {
    // ---------------------------------------------------------------- activation producer: token codes and their scales.
    // Its own thread, because the fences a GEMM2 unit needs (acquire, then generic -> async proxy) must not sit in the
    // thread that keeps the weight stream full.
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true, have_next = false;
      int next_count = 0;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        const bool second = u >= units1;
        const int v = second ? u - units1 : u;
        const int tiles_m = second ? kW2Tiles : kW13Tiles, tiles_k = second ? kK2Tiles : kK1Tiles;
        const int b = v / tiles_m;
        const uint8_t* sfb_src = second ? ep.sfh + static_cast<int64_t>(b) * C2::kActAtomsPerBlock * kAtomBytes
                                        : sf_x + static_cast<int64_t>(b) * C::kActAtomsPerBlock * kAtomBytes;
        if (second) {
          // h of this row block must be complete and visible to the copy engine before it is read. The count was
          // fetched while the previous unit's copies were issued, so the usual case costs no memory round trip.
          // Usual case: the look-ahead (an acquire load: a load, not a fence, so it does not wait for this thread's
          // copies in flight) has already seen 12. The writers ordered their stores for the copy engine before they
          // counted (see the GEMM1 epilogue), so no fence is needed here.
          if (!(have_next && next_count >= kW13Tiles)) {
            if (!wait_count(done + b, kW13Tiles, abort_v, status)) { ok = false; break; }
            asm volatile("fence.proxy.async;" ::: "memory");
          }
        }
        for (int kt = 0; kt < tiles_k; ++kt, ++it) {
          const uint32_t s = it % CC::kStages, ph = (it / CC::kStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_v, status)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t base = tiles + s * C::kStageBytes;
          tma_load_2d(base + C::kBOffset, second ? &map_h : &map_x, kt * 128, b * BM, full);
          bulk_load(base + C::kSfbOffset, sfb_src + kt * C::kSfBytes, C::kSfBytes, full);
        }
        const int un = u + static_cast<int>(gridDim.x);  // look ahead: the next unit's completion count
        have_next = un < total_units && un >= units1;
        if (have_next)
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(next_count) : "l"(done + (un - units1) / kW2Tiles) : "memory");
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BM >> 3) << 17) | (1u << 23) | (8u << 24);
      constexpr uint32_t kId0 = kIdesc, kId1 = kIdesc | (2u << 29) | (2u << 4);
      // as in grouped_gemm_kernel: warp 7 copies the scales, this thread waits for that and issues the MMAs
      const uint32_t sf0 = smem_u32(&bar_sf[0]), empty0 = smem_u32(&bar_empty[0]);
      uint32_t slot = 0, ph = 0, sfset = 0, ui = 0;
      uint32_t lo = tiles >> 4, sf = sf0, empty = empty0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x, ++ui) {
        const int tiles_k = u >= units1 ? kK2Tiles : kK1Tiles;
        const uint32_t acc = ui & 1u, aph = (ui >> 1) & 1u;
        if (!mbar_wait(smem_u32(&bar_tempty[acc]), aph ^ 1u, abort_v, status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::kAccCols;
        for (int kt = 0; kt < tiles_k; ++kt) {
          if (!mbar_wait(sf, ph, abort_v, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t t_sfa = tmem_base + C::kSfaCol + 16u * sfset, t_sfb = t_sfa + 8u;
          const uint32_t w_lo = lo, x_lo = lo + (C::kBOffset >> 4);
          tc_mma_mxf4_lo<2>(d_tmem, w_lo, x_lo, kId0, t_sfa, t_sfb, static_cast<uint32_t>(kt != 0));
          tc_mma_mxf4_lo<1>(d_tmem, w_lo + 2, x_lo + 2, kId1, t_sfa, t_sfb);
          tc_mma_mxf4_lo<1>(d_tmem, w_lo + 4, x_lo + 4, kId0, t_sfa + 4, t_sfb + 4);
          tc_mma_mxf4_lo<1>(d_tmem, w_lo + 6, x_lo + 6, kId1, t_sfa + 4, t_sfb + 4);
          tc_commit(empty);
          sfset = (sfset + 1u) & (C::kSfSets - 1);
          if (++slot == CC::kStages) {
            slot = 0; ph ^= 1u; lo = tiles >> 4; sf = sf0; empty = empty0;
          } else {
            lo += C::kStageBytes >> 4; sf += 8; empty += 8;
          }
        }
        if (ok) tc_commit(smem_u32(&bar_tfull[acc]));
      }
      if (*abort_v) drain_tcgen05(smem_u32(&bar_drain[0]));
    }
  } else if (warp == 7) {
    // ---------------------------------------------------------------- scale copies: shared memory -> tensor memory
    if (lane == 0) {
      const uint32_t full0 = smem_u32(&bar_full[0]), sf0 = smem_u32(&bar_sf[0]);
      uint32_t slot = 0, ph = 0, sfset = 0;
      uint32_t lo = tiles >> 4, full = full0, sf = sf0;
      bool ok = true;
      for (int u = blockIdx.x; u < total_units && ok; u += gridDim.x) {
        const int tiles_k = u >= units1 ? kK2Tiles : kK1Tiles;
        for (int kt = 0; kt < tiles_k; ++kt) {
          if (!mbar_wait(full, ph, abort_v, status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t t_sfa = tmem_base + C::kSfaCol + 16u * sfset, t_sfb = t_sfa + 8u;
          tc_cp_scales_lo(t_sfa, lo + (C::kABytes >> 4));
          tc_cp_scales_lo(t_sfa + 4, lo + ((C::kABytes + kAtomBytes) >> 4));
          tc_cp_scales_lo(t_sfb, lo + (C::kSfbOffset >> 4));
          tc_cp_scales_lo(t_sfb + 4, lo + ((C::kSfbOffset + kAtomBytes) >> 4));
          tc_commit(sf);
          sfset = (sfset + 1u) & (C::kSfSets - 1);
          if (++slot == CC::kStages) {
            slot = 0; ph ^= 1u; lo = tiles >> 4; full = full0; sf = sf0;
          } else {
            lo += C::kStageBytes >> 4; full += 8; sf += 8;
          }
        }
      }
      if (*abort_v) drain_tcgen05(smem_u32(&bar_drain[1]));
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    float* stage_f = reinterpret_cast<float*>(smem_raw + (tiles - smem_u32(smem_raw)) + CC::kStages * C::kStageBytes);
    uint32_t ui = 0;
    bool have_ahead = false;
    int ahead_sid = 0;
    float ahead_wt = 0.0f;
    for (int u = blockIdx.x; u < total_units; u += gridDim.x, ++ui) {
      const bool second = u >= units1;
      const int v = second ? u - units1 : u;
      const int tiles_m = second ? kW2Tiles : kW13Tiles;
      const int b = v / tiles_m, mt = v % tiles_m;
      const uint32_t acc = ui & 1u, aph = (ui >> 1) & 1u;
      const int64_t row0 = static_cast<int64_t>(b) * BM;
      if (second && et < BM) {
        if (!have_ahead) {
          ahead_sid = __ldcg(sorted_ids + row0 + et);
          ahead_wt = __ldcg(sorted_w + row0 + et);
        }
        s_dst[et] = placer.row(ahead_sid);
        s_wt[et] = ahead_wt;
      }
      if (!epilogue_all(mbar_wait(smem_u32(&bar_tfull[acc]), aph, abort_v, status), 1u)) break;
      tc_fence_after();
      {  // look ahead: the rows of this CTA's next unit, when that is a GEMM2 unit
        const int un = u + static_cast<int>(gridDim.x);
        have_ahead = un < total_units && un >= units1;
        if (have_ahead && et < BM) {
          const int64_t r1 = static_cast<int64_t>((un - units1) / kW2Tiles) * BM + et;
          ahead_sid = __ldcg(sorted_ids + r1);
          ahead_wt = __ldcg(sorted_w + r1);
        }
      }
      const uint32_t t_acc = tmem_base + acc * C::kAccCols + (static_cast<uint32_t>(q * 32) << 16);
      if (!second) {
        float* mine = stage_f + (q >> 1) * 68 + (q & 1) * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BM; c0 += C::kEpiCols) {
#pragma unroll 1
          for (int cc = 0; cc < C::kEpiCols; cc += 16) {
            uint32_t vv[16];
            tc_ld16(t_acc + c0 + cc, vv);
#pragma unroll
            for (int j = 0; j < 16; ++j) mine[(cc + j) * C::kEpiRowFloats] = __uint_as_float(vv[j]);
          }
          if (c0 + C::kEpiCols >= BM) {
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_tempty[acc]));
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          for (int item = et; item < 2 * C::kEpiCols; item += 128) {
            const int j = item >> 1, g = item & 1;
            const float4* src = reinterpret_cast<const float4*>(stage_f + j * C::kEpiRowFloats + g * 68);
            float h[32];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float4 gv = src[k], uv = src[8 + k];
              h[4 * k + 0] = swiglu_oai(gv.x, uv.x);
              h[4 * k + 1] = swiglu_oai(gv.y, uv.y);
              h[4 * k + 2] = swiglu_oai(gv.z, uv.z);
              h[4 * k + 3] = swiglu_oai(gv.w, uv.w);
            }
            float amax = 0.0f;
#pragma unroll
            for (int k = 0; k < 32; ++k) amax = fmaxf(amax, fabsf(h[k]));
            const int sc = quark_even_e8m0(amax);
            const float inv = __uint_as_float(static_cast<uint32_t>(254 - sc) << 23);
            uint32_t words[4];
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
              uint32_t acc_w = 0;
#pragma unroll
              for (int k = 0; k < 4; ++k)
                acc_w |= cvt_e2m1x2(h[8 * wd + 2 * k] * inv, h[8 * wd + 2 * k + 1] * inv) << (8 * k);
              words[wd] = acc_w;
            }
            const int grp = 2 * mt + g;
            const int n = c0 + j;
            *reinterpret_cast<uint4*>(ep.hq + (row0 + n) * (kI / 2) + grp * 16) =
                make_uint4(words[0], words[1], words[2], words[3]);
            ep.sfh[(static_cast<int64_t>(b) * (kI / 128) + (grp >> 2)) * kAtomBytes + atom_offset(n, grp & 3)] =
                static_cast<uint8_t>(sc);
          }
          // this thread's h stores: ordered for the copy engine (async proxy) and visible device-wide before the count moves
          asm volatile("fence.proxy.async;" ::: "memory");
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if (et == 0) atomicAdd(done + b, 1);  // one more GEMM1 tile of row block b is complete
      } else {
        float* mine = stage_f + q * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BM; c0 += C2::kOutCols) {
#pragma unroll
          for (int cc = 0; cc < C2::kOutCols; cc += 16) {
            uint32_t vv[16];
            tc_ld16(t_acc + c0 + cc, vv);
#pragma unroll
            for (int j = 0; j < 16; ++j) mine[(cc + j) * C2::kOutRowFloats] = __uint_as_float(vv[j]);
          }
          if (c0 + C2::kOutCols >= BM) {
            tc_fence_before();
            mbar_arrive(smem_u32(&bar_tempty[acc]));
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll 2
          for (int item = et; item < C2::kOutCols * 32; item += 128) {
            const int j = item >> 5, seg = item & 31;
            __nv_bfloat16* row_dst = s_dst[c0 + j];
            if (row_dst != nullptr) {
              const float s_w = s_wt[c0 + j];
              const float4 x4 = *reinterpret_cast<const float4*>(stage_f + j * C2::kOutRowFloats + seg * 4);
              const __nv_bfloat162 lo = __floats2bfloat162_rn(x4.x * s_w, x4.y * s_w);
              const __nv_bfloat162 hi = __floats2bfloat162_rn(x4.z * s_w, x4.w * s_w);
              uint2 packed;
              packed.x = *reinterpret_cast<const uint32_t*>(&lo);
              packed.y = *reinterpret_cast<const uint32_t*>(&hi);
              *reinterpret_cast<uint2*>(row_dst + mt * 128 + seg * 4) = packed;
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
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

// ------------------------------------------------------------------------------------------------ host side
constexpr int64_t kWideFromRows = 20000;  // sorted rows (about 3000 tokens) from which GEMM1 uses 256 weight rows per MMA
template <int MODE, int BM>
static int launch(const CUtensorMap& mx, const uint8_t* w_tiles, const uint8_t* sf_x,
                  const int32_t* block_expert, const int32_t* num_valid, const EpilogueArgs& ep, int64_t max_rows,
                  int num_experts, int32_t* status, cudaStream_t stream) {
  using C = Cfg<MODE, BM>;
  static PerDeviceOnce once;
  const int rc = once.run([] {
    return static_cast<int>(cudaFuncSetAttribute(grouped_gemm_kernel<MODE, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 C::kSmemBytes));
  });
  if (rc) return rc;
  const int64_t max_units = max_rows / BM * C::kTilesM;
  const int64_t ctas = sm_count();
  int grid = static_cast<int>(max_units < ctas ? max_units : ctas);
  if (ep.max_ctas > 0 && grid > ep.max_ctas) grid = ep.max_ctas;
  if (grid <= 0) return 0;
  B200MOE_LAUNCH((grouped_gemm_kernel<MODE, BM>), grid, C::kThreads, C::kSmemBytes, stream, mx, w_tiles, sf_x, block_expert, num_valid, ep, status, num_experts, static_cast<int>(max_rows / BM));
  return 0;
}

template <int MODE>
static int launch_bm(int bm, const CUtensorMap& mx, const uint8_t* w_tiles, const uint8_t* sf_x,
                     const int32_t* block_expert, const int32_t* num_valid, const EpilogueArgs& ep, int64_t max_rows,
                     int num_experts, int32_t* status, cudaStream_t stream) {
  switch (bm) {
    case 16: return launch<MODE, 16>(mx, w_tiles, sf_x, block_expert, num_valid, ep, max_rows, num_experts, status, stream);
    case 32: return launch<MODE, 32>(mx, w_tiles, sf_x, block_expert, num_valid, ep, max_rows, num_experts, status, stream);
    case 64: return launch<MODE, 64>(mx, w_tiles, sf_x, block_expert, num_valid, ep, max_rows, num_experts, status, stream);
    case 128:
      return launch<MODE, 128>(mx, w_tiles, sf_x, block_expert, num_valid, ep, max_rows, num_experts, status, stream);
  }
  return B200MOE_E_ARG;
}


template <int BM>
static int launch12(const CUtensorMap& mx, const CUtensorMap& mh, const uint8_t* w13t, const uint8_t* w2t,
                    const uint8_t* sfx, const int32_t* block_expert, const int32_t* num_valid, const EpilogueArgs& ep,
                    int32_t* done, int64_t max_rows, int num_experts, int32_t* status, cudaStream_t stream) {
  using CC = Cfg12<BM>;
  static PerDeviceOnce once;
  const int rc = once.run([] {
    return static_cast<int>(cudaFuncSetAttribute(gemm12_kernel<BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, CC::kSmemBytes));
  });
  if (rc) return rc;
  const int64_t max_units = max_rows / BM * (kW13Tiles + kW2Tiles);
  const int grid = static_cast<int>(max_units < sm_count() ? max_units : sm_count());
  if (grid <= 0) return 0;
  B200MOE_LAUNCH((gemm12_kernel<BM>), grid, 256, CC::kSmemBytes, stream, mx, mh, w13t, w2t, sfx, block_expert, num_valid, ep,
                 done, status, num_experts, static_cast<int>(max_rows / BM));
  return 0;
}

int set_wait_limit_routed(unsigned long long ns) { return set_wait_limit_here(ns); }

}  // namespace b200moe

extern "C" int b200moe_gemm12(const uint8_t* w13t, const uint8_t* w2t, int num_experts, const uint8_t* xq_sorted,
                              const uint8_t* sfx, const int32_t* block_expert, const int32_t* num_valid,
                              const int32_t* sorted_ids, const float* sorted_w, int64_t max_rows, int bm, int64_t tokens,
                              uint8_t* hq, uint8_t* sfh, int32_t* done, void* slots_bf16, int32_t* status, void* stream) {
  using namespace b200moe;
  if (!w13t || !w2t || !xq_sorted || !sfx || !block_expert || !num_valid || !sorted_ids || !sorted_w || !hq || !sfh ||
      !done || !slots_bf16 || !status)
    return B200MOE_E_ARG;
  if (num_experts < 1 || num_experts > kMaxE || max_rows < 0 || tokens < 0 || (bm != 16 && bm != 32 && bm != 64) ||
      max_rows % bm)
    return B200MOE_E_ARG;
  if (misaligned(w13t, 16) || misaligned(w2t, 16) || misaligned(xq_sorted, 16) || misaligned(sfx, 16) ||
      misaligned(hq, 16) || misaligned(sfh, 16))
    return B200MOE_E_ALIGN;
  if (max_rows == 0) return 0;
  CUtensorMap mx, mh;
  int r = make_map(&mx, xq_sorted, kH / 2, static_cast<uint64_t>(max_rows), static_cast<uint32_t>(bm));
  if (r) return r;
  r = make_map(&mh, hq, kI / 2, static_cast<uint64_t>(max_rows), static_cast<uint32_t>(bm));
  if (r) return r;
  EpilogueArgs ep{};
  ep.hq = hq;
  ep.sfh = sfh;
  ep.sorted_ids = sorted_ids;
  ep.sorted_w = sorted_w;
  ep.slots = static_cast<__nv_bfloat16*>(slots_bf16);
  ep.tokens = tokens;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (bm) {
    case 16: return launch12<16>(mx, mh, w13t, w2t, sfx, block_expert, num_valid, ep, done, max_rows, num_experts, status, st);
    case 32: return launch12<32>(mx, mh, w13t, w2t, sfx, block_expert, num_valid, ep, done, max_rows, num_experts, status, st);
    case 64: return launch12<64>(mx, mh, w13t, w2t, sfx, block_expert, num_valid, ep, done, max_rows, num_experts, status, st);
  }
  return B200MOE_E_ARG;
}

extern "C" int b200moe_gemm1_swiglu_quant(const uint8_t* w13t, int num_experts, const uint8_t* xq_sorted,
                                          const uint8_t* sfx, const int32_t* block_expert, const int32_t* num_valid,
                                          int64_t max_rows, int bm, uint8_t* hq, uint8_t* sfh,
                                          const uint8_t* prefetch_w2t, int32_t* status, void* stream) {
  using namespace b200moe;
  if (!w13t || !xq_sorted || !sfx || !block_expert || !num_valid || !hq || !sfh || !status) return B200MOE_E_ARG;
  if (num_experts < 1 || num_experts > kMaxE || max_rows < 0 || (bm != 16 && bm != 32 && bm != 64 && bm != 128) ||
      max_rows % bm)
    return B200MOE_E_ARG;
  if (misaligned(w13t, 16) || misaligned(xq_sorted, 16) || misaligned(sfx, 16) || misaligned(hq, 16) ||
      misaligned(sfh, 16))
    return B200MOE_E_ALIGN;
  if (max_rows == 0) return 0;
  // Prefill sizes: 256 weight rows per MMA on one CTA (twice the math per issued instruction). Measured, GEMM1 alone, us:
  // 4096 tokens 127 (128-column kernel 129), 8192 tokens 183 (197; CTA pairs 199), 16384 tokens 312 (320; pairs 320).
  if (bm == 128 && max_rows >= kWideFromRows)
    return b200moe_gemm1_swiglu_quant_wide(w13t, num_experts, xq_sorted, sfx, block_expert, num_valid, max_rows, hq, sfh,
                                           status, stream);
  CUtensorMap mx;
  const int r = make_map(&mx, xq_sorted, kH / 2, static_cast<uint64_t>(max_rows), static_cast<uint32_t>(bm));
  if (r) return r;
  EpilogueArgs ep{};
  ep.hq = hq;
  ep.sfh = sfh;
  ep.next_tiles = misaligned(prefetch_w2t, 16) ? nullptr : prefetch_w2t;
  return launch_bm<1>(bm, mx, w13t, sfx, block_expert, num_valid, ep, max_rows, num_experts, status,
                      static_cast<cudaStream_t>(stream));
}

static int gemm2_common(const uint8_t* w2t, int num_experts, const uint8_t* hq, const uint8_t* sfh,
                        const int32_t* block_expert, const int32_t* num_valid, const int32_t* sorted_ids,
                        const float* sorted_w, int64_t max_rows, int bm, int64_t tokens, b200moe::EpilogueArgs ep,
                        int32_t* status, void* stream) {
  using namespace b200moe;
  if (!w2t || !hq || !sfh || !block_expert || !num_valid || !sorted_ids || !sorted_w || !status) return B200MOE_E_ARG;
  if (num_experts < 1 || num_experts > kMaxE || max_rows < 0 || tokens < 0 ||
      (bm != 16 && bm != 32 && bm != 64 && bm != 128) || max_rows % bm)
    return B200MOE_E_ARG;
  if (misaligned(w2t, 16) || misaligned(hq, 16) || misaligned(sfh, 16)) return B200MOE_E_ALIGN;
  if (max_rows == 0) return 0;
  CUtensorMap mx;
  const int r = make_map(&mx, hq, kI / 2, static_cast<uint64_t>(max_rows), static_cast<uint32_t>(bm));
  if (r) return r;
  ep.sorted_ids = sorted_ids;
  ep.sorted_w = sorted_w;
  ep.tokens = tokens;
  return launch_bm<2>(bm, mx, w2t, sfh, block_expert, num_valid, ep, max_rows, num_experts, status,
                      static_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_gemm2_weighted(const uint8_t* w2t, int num_experts, const uint8_t* hq, const uint8_t* sfh,
                                      const int32_t* block_expert, const int32_t* num_valid, const int32_t* sorted_ids,
                                      const float* sorted_w, int64_t max_rows, int bm, int64_t tokens, void* slots_bf16,
                                      int32_t* status, void* stream) {
  if (!slots_bf16) return B200MOE_E_ARG;
  b200moe::EpilogueArgs ep{};
  ep.slots = static_cast<__nv_bfloat16*>(slots_bf16);
  return gemm2_common(w2t, num_experts, hq, sfh, block_expert, num_valid, sorted_ids, sorted_w, max_rows, bm, tokens, ep,
                      status, stream);
}

extern "C" int b200moe_gemm2_weighted_peer_range(const uint8_t* w2t, int num_experts, const uint8_t* hq, const uint8_t* sfh,
                                           const int32_t* block_expert, const int32_t* num_valid,
                                           const int32_t* sorted_ids, const float* sorted_w, int64_t max_rows, int bm,
                                           int64_t tokens, const int32_t* row_rank, const int32_t* row_pair,
                                           void* const* peer_slots, int world, int64_t peer_rows,
                                           const int32_t* block_range, int max_ctas, int32_t* status, void* stream) {
  if (!row_rank || !row_pair || !peer_slots || world < 1 || world > 8 || peer_rows < 1 || !status) return B200MOE_E_ARG;
  b200moe::EpilogueArgs ep{};
  for (int r = 0; r < 8; ++r) {
    ep.peer_slots[r] = static_cast<__nv_bfloat16*>(peer_slots[r < world ? r : 0]);
    if (!ep.peer_slots[r] || (reinterpret_cast<uintptr_t>(ep.peer_slots[r]) & 15)) return B200MOE_E_ARG;
  }
  ep.row_rank = row_rank;
  ep.row_pair = row_pair;
  ep.world = world;
  ep.peer_rows = peer_rows;
  ep.status = status;
  ep.block_range = block_range;
  ep.max_ctas = max_ctas;
  return gemm2_common(w2t, num_experts, hq, sfh, block_expert, num_valid, sorted_ids, sorted_w, max_rows, bm, tokens, ep,
                      status, stream);
}

extern "C" int b200moe_gemm2_weighted_peer(const uint8_t* w2t, int num_experts, const uint8_t* hq, const uint8_t* sfh,
                                           const int32_t* block_expert, const int32_t* num_valid,
                                           const int32_t* sorted_ids, const float* sorted_w, int64_t max_rows, int bm,
                                           int64_t tokens, const int32_t* row_rank, const int32_t* row_pair,
                                           void* const* peer_slots, int world, int64_t peer_rows, int32_t* status,
                                           void* stream) {
  return b200moe_gemm2_weighted_peer_range(w2t, num_experts, hq, sfh, block_expert, num_valid, sorted_ids, sorted_w, max_rows,
                                           bm, tokens, row_rank, row_pair, peer_slots, world, peer_rows, nullptr, 0, status,
                                           stream);
}
