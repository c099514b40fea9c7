// Device-side primitives for kernels that talk to peer GPUs through a symmetric heap.
//
// A symmetric buffer is the same allocation made on every rank; every rank maps every peer's
// copy (CUDA IPC), so a kernel addresses "rank p's copy" through a pointer table.  Cross-rank
// ordering uses flag words in the peers' memory: a rank publishes `epoch` into slot [my_rank]
// of every peer's flag array with a system-scope release store and waits, with a time limit,
// until every slot of its own array has reached `epoch` (system-scope acquire loads).
// A wait that runs out records kStatusPeerWaitTimeout and returns false; the caller then skips
// the rest of its work and the kernel returns normally, so the context stays usable and the
// host can turn the status into a communicator error.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common.cuh"

namespace ferrl {

constexpr int kMaxRanks = 16;

struct PeerTable {
  void* ptr[kMaxRanks];
};

#ifdef __CUDACC__
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Called by ONE thread. flags[p] is rank p's flag array (kMaxRanks words per barrier slot).
__device__ __forceinline__ bool peer_barrier(const PeerTable& flags, int slot, int rank, int world, uint32_t epoch,
                                             uint64_t limit_ns, int* status) {
  __threadfence_system();
  for (int p = 0; p < world; ++p)
    st_release_sys(static_cast<uint32_t*>(flags.ptr[p]) + slot * kMaxRanks + rank, epoch);
  const uint32_t* mine = static_cast<const uint32_t*>(flags.ptr[rank]) + slot * kMaxRanks;
  const uint64_t t0 = globaltimer_ns();
  for (int p = 0; p < world; ++p) {
    uint32_t spins = 0;
    // epochs only grow; signed distance tolerates wrap-around
    while (static_cast<int32_t>(ld_acquire_sys(mine + p) - epoch) < 0) {
      if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > limit_ns) {
        atomicCAS(status, kStatusOk, kStatusPeerWaitTimeout);
        return false;
      }
    }
  }
  __threadfence_system();
  return true;
}
#endif

}  // namespace ferrl
