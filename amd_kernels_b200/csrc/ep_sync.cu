// Expert parallel: ordering the ranks of a node without a collective library call.
//
// Between the phases of the expert-parallel step (send plan -> push of the quantised rows -> grouped GEMMs with the combine
// in GEMM2's epilogue -> reduce) every rank has to know that every other rank's stores into its buffers have landed. One
// launch of this kernel per ordering point does it over the peer mappings the step uses anyway: thread r stores this rank's
// epoch into slot `rank` of peer r's flag array (after a system-scope fence, so that everything this rank stored before is
// visible first) and then waits, bounded, until slot r of its own flag array has reached the epoch. Optionally the launch
// also carries a payload: this rank's row of the W x W matrix of row counts, stored into every peer's copy of the matrix
// before the flag (the all-gather of the send plan). Measured at 4 ranks, the three small NCCL collectives this replaces
// took 37 + 19..47 + 16..24 us of a 570 us step.
//
// The epoch is a device counter local to the rank, advanced by the kernel itself, so the launch can sit in a CUDA graph;
// the ranks stay in step because they make the same sequence of calls. Flags only grow, so a peer that is already one
// ordering point ahead does no harm. A wait that runs out (a rank that died or fell out of step) records
// B200MOE_DEV_TIMEOUT in the status word and the kernel returns; nothing traps.
#include "tc_ptx.cuh"

namespace b200moe {

struct PeerTable {
  void* p[8];
};

__global__ void __launch_bounds__(32) ep_sync_kernel(PeerTable flags, PeerTable matrices, const int64_t* __restrict__ my_counts,
                                                     int world, int rank, int32_t* __restrict__ epoch_counter,
                                                     int32_t* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();  // everything this rank launched before has completed, its stores are performed
  launder(my_counts);
  launder(epoch_counter);
  const int r = static_cast<int>(threadIdx.x);
  const int32_t epoch = __ldcg(epoch_counter) + 1;
  if (r < world) {
    if (my_counts != nullptr && matrices.p[r] != nullptr) {
      int64_t* row = static_cast<int64_t*>(matrices.p[r]) + static_cast<int64_t>(rank) * world;
      for (int d = 0; d < world; ++d) row[d] = __ldcg(my_counts + d);
    }
    __threadfence_system();
    int32_t* theirs = static_cast<int32_t*>(flags.p[r]) + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
    const int32_t* mine = static_cast<const int32_t*>(flags.p[rank]) + r;
    const uint64_t t0 = global_timer(), limit = wait_limit_ns();
    uint32_t spins = 0;
    while (true) {
      int32_t seen;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (seen - epoch >= 0) break;  // flags only grow (compared as a difference: the counter may wrap)
      if ((++spins & 15u) == 0u && global_timer() - t0 > limit) {
        atomicExch(status, B200MOE_DEV_TIMEOUT);
        break;
      }
    }
  }
  __syncwarp();
  if (r == 0) *epoch_counter = epoch;
}

int set_wait_limit_ep_sync(unsigned long long ns) { return set_wait_limit_here(ns); }

}  // namespace b200moe

extern "C" int b200moe_ep_sync(void* const* peer_flags, void* const* peer_matrices, const int64_t* my_counts, int world,
                               int rank, int32_t* epoch_counter, int32_t* status, void* stream) {
  using namespace b200moe;
  if (!peer_flags || !epoch_counter || !status || world < 1 || world > 8 || rank < 0 || rank >= world) return B200MOE_E_ARG;
  if ((my_counts != nullptr) != (peer_matrices != nullptr)) return B200MOE_E_ARG;
  PeerTable f{}, m{};
  for (int r = 0; r < world; ++r) {
    f.p[r] = peer_flags[r];
    if (!f.p[r] || (reinterpret_cast<uintptr_t>(f.p[r]) & 3)) return B200MOE_E_ARG;
    if (peer_matrices) {
      m.p[r] = peer_matrices[r];
      if (!m.p[r] || (reinterpret_cast<uintptr_t>(m.p[r]) & 7)) return B200MOE_E_ARG;
    }
  }
  B200MOE_LAUNCH(ep_sync_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), f, m, my_counts, world, rank, epoch_counter,
                 status);
  return 0;
}
