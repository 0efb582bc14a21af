// PTX wrappers shared by the tensor-core kernels (sm_100a): mbarriers with bounded waits, TMA / bulk copies, tcgen05
// alloc / cp / mma / ld / commit, shared-memory and scale descriptors.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace b200moe {

// ------------------------------------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// How long a device-side wait may last before the kernel gives up (status B200MOE_DEV_TIMEOUT). Every translation
// unit that includes this header carries its own copy; b200moe_set_wait_limit_ns updates all of them on the current
// device. Read only on the slow path of a wait.
static __device__ unsigned long long g_wait_limit_ns = 2000000000ull;
__device__ __forceinline__ uint64_t wait_limit_ns() {
  return *reinterpret_cast<volatile unsigned long long*>(&g_wait_limit_ns);
}
static inline int set_wait_limit_here(unsigned long long ns) {
  return static_cast<int>(cudaMemcpyToSymbol(g_wait_limit_ns, &ns, sizeof(ns)));
}

// Bounded wait. Returns false when the CTA is aborting (this wait or another one ran out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
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

// After an abort: let the copies of the last `stages` pipeline slots land (one overall limit, not one per slot) before
// the CTA gives up its shared memory. `it` = stages issued so far.
__device__ __forceinline__ void drain_copies(const uint64_t* bar_full, uint32_t it, uint32_t stages) {
  const uint32_t pending = it < stages ? it : stages;
  const uint64_t t0 = global_timer(), limit = wait_limit_ns();
  for (uint32_t j = 0; j < pending; ++j) {
    const uint32_t idx = it - 1 - j, s = idx % stages, ph = (idx / stages) & 1u;
    while (!mbar_try_wait(static_cast<uint32_t>(__cvta_generic_to_shared(bar_full + s)), ph) && global_timer() - t0 < limit) {}
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// After an abort: wait (bounded) until every tcgen05 operation this thread issued has completed, so tensor memory is
// not freed under an MMA or a scale copy still in flight. `bar` is a barrier nothing else uses (count 1, phase 0).
__device__ __forceinline__ void drain_tcgen05(uint32_t bar) {
  tc_commit(bar);
  const uint64_t t0 = global_timer(), limit = wait_limit_ns();
  while (!mbar_try_wait(bar, 0) && global_timer() - t0 < limit) {}
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]),
        "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]),
        "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// the same load without the wait: issue several, then one tcgen05.wait::ld
__device__ __forceinline__ void tc_ld32_nowait(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
      "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]),
        "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]),
        "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// AND of a predicate over the 128 threads of one epilogue group (named barrier 1 or 2); every one of them gets the result.
__device__ __forceinline__ bool epilogue_all(bool ok, uint32_t barrier_id) {
  uint32_t out;
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.and.pred p, %2, 128, q;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(ok)), "r"(barrier_id)
      : "memory");
  return out != 0;
}

// Shared-memory descriptors are passed as their low 32-bit word (shared-memory address >> 4; the tiles sit below 256 KB,
// so it fits 14 bits) and the constant high word is an immediate: the instruction stream of the issuing threads bounds
// the kernels, so no 64-bit arithmetic is left in their loops. Operand tiles are K-major with 128-byte rows and the
// 128-byte swizzle (8-row groups 1024 bytes apart); a scale atom is 32 rows of 16 bytes, no swizzle (8-row groups 128
// bytes apart).
constexpr uint32_t kOperandDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024 B, version bit 46, 128B swizzle
constexpr uint32_t kScaleDescHi = (128u >> 4) | (1u << 14);                  // SBO 128 B, version bit 46, no swizzle

__device__ __forceinline__ void tc_cp_scales_lo(uint32_t taddr, uint32_t desc_lo) {
  asm volatile("{\n.reg .b64 d;\nmov.b64 d, {%1, %2};\ntcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n}\n" ::"r"(taddr),
               "r"(desc_lo), "n"(kScaleDescHi)
               : "memory");
}
// ACC: 1 = accumulate, 0 = overwrite, 2 = take it from `accumulate`
template <int ACC>
__device__ __forceinline__ void tc_mma_mxf4_lo(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t sfa,
                                               uint32_t sfb, uint32_t accumulate = 1u) {
  if (ACC == 2) {
    asm volatile(
        "{\n.reg .b64 da, db;\n.reg .pred p;\nmov.b64 da, {%1, %7};\nmov.b64 db, {%2, %7};\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %3, [%4], [%5], p;\n}\n" ::"r"(d),
        "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate), "n"(kOperandDescHi)
        : "memory");
  } else {
    asm volatile(
        "{\n.reg .b64 da, db;\n.reg .pred p;\nmov.b64 da, {%1, %6};\nmov.b64 db, {%2, %6};\nsetp.ne.b32 p, %7, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %3, [%4], [%5], p;\n}\n" ::"r"(d),
        "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(sfa), "r"(sfb), "n"(kOperandDescHi), "n"(ACC)
        : "memory");
  }
}

// block-scaled FP8 (E4M3 x E4M3, one UE8M0 scale per 32 elements): M = 128, K = 32 per instruction
template <int ACC>
__device__ __forceinline__ void tc_mma_mxf8_lo(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t sfa,
                                               uint32_t sfb, uint32_t accumulate = 1u) {
  if (ACC == 2) {
    asm volatile(
        "{\n.reg .b64 da, db;\n.reg .pred p;\nmov.b64 da, {%1, %7};\nmov.b64 db, {%2, %7};\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, %3, [%4], [%5], p;\n}\n" ::"r"(d),
        "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate), "n"(kOperandDescHi)
        : "memory");
  } else {
    asm volatile(
        "{\n.reg .b64 da, db;\n.reg .pred p;\nmov.b64 da, {%1, %6};\nmov.b64 db, {%2, %6};\nsetp.ne.b32 p, %7, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, %3, [%4], [%5], p;\n}\n" ::"r"(d),
        "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(sfa), "r"(sfb), "n"(kOperandDescHi), "n"(ACC)
        : "memory");
  }
}



}  // namespace b200moe
