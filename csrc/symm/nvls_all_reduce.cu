// All-reduce through NVSwitch multicast (NVLS): the sum is formed inside the switch.
//
// The buffer is a symmetric allocation bound to a multicast object, so one address (`mc`) names every
// rank's copy at once: `multimem.ld_reduce` on it returns the sum of all copies, computed by the switch,
// and `multimem.st` writes a value into all copies.  Two shots, so that every rank ends with the same
// bits: after a barrier, rank r reduces slice r of the buffer with `multimem.ld_reduce` (fp32
// accumulation for bf16) and broadcasts the result into all copies with `multimem.st`; after a second
// barrier every rank copies its now complete local copy to the output.  Per rank n / world elements
// cross NVLink in each direction, against (world - 1) n / world for the plain peer-load form in
// csrc/dp/dp_step.cu (`symm_all_reduce_kernel`) - the reference's counterpart is a blocking
// ncclAllReduce per activation (crates/ferrl/src/tensor_parallel.rs:417-510).
//
// The barriers are the flag words of the symmetric heap (plain peer stores, bounded waits that leave a
// status word); only the data path uses the multicast address.  A rank must never exit while peers
// still use the multicast object: the heap's owner tears the group down collectively.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"
#include "symm.cuh"

namespace cg = cooperative_groups;

namespace ferrl {
namespace {

template <typename T> __device__ __forceinline__ uint4 mc_ld_reduce(const void* mc);
template <> __device__ __forceinline__ uint4 mc_ld_reduce<__nv_bfloat16>(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
template <> __device__ __forceinline__ uint4 mc_ld_reduce<float>(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void mc_st(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// n16: number of 16-byte units, a multiple of `world`
template <typename T>
__global__ void __launch_bounds__(512)
nvls_all_reduce_kernel(uint4* mc, const uint4* __restrict__ local, PeerTable flags, uint4* __restrict__ out, long long n16,
                       int rank, int world, uint32_t epoch, uint64_t limit_ns, int* status, int* abort_word) {
  cg::grid_group grid = cg::this_grid();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const bool ok = peer_barrier(flags, 4, rank, world, epoch, limit_ns, status);      // every rank has staged its input
    *abort_word = ok ? 0 : 1;
    __threadfence();
  }
  grid.sync();
  if (*reinterpret_cast<volatile int*>(abort_word)) return;
  const long long per = n16 / world, lo = per * rank;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  // four requests in flight per thread: the round trip through the switch is long
  constexpr int U = 4;
  long long i = lo + tid;
  for (; i + (U - 1) * nthreads < lo + per; i += U * nthreads) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = mc_ld_reduce<T>(mc + i + u * nthreads);
#pragma unroll
    for (int u = 0; u < U; ++u) mc_st(mc + i + u * nthreads, v[u]);
  }
  for (; i < lo + per; i += nthreads) {
    const uint4 v = mc_ld_reduce<T>(mc + i);
    mc_st(mc + i, v);
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const bool ok = peer_barrier(flags, 5, rank, world, epoch, limit_ns, status);      // every slice is reduced and broadcast
    if (!ok) *abort_word = 1;
    __threadfence();
  }
  grid.sync();
  if (*reinterpret_cast<volatile int*>(abort_word)) return;
  for (long long j = tid; j < n16; j += nthreads) out[j] = local[j];
}

}  // namespace

const char* nvls_all_reduce(int dtype, void* mc, const void* local, const PeerTable& flags, void* out, long long nbytes, int rank,
                            int world, unsigned epoch, unsigned long long limit_ns, int* status, int* abort_word, int num_sms,
                            cudaStream_t s) {
  if (world < 1 || world > kMaxRanks) return "nvls_all_reduce: world size out of range";
  if (nbytes == 0) return nullptr;
  if (nbytes % (16LL * world)) return "nvls_all_reduce: byte count must be a multiple of 16 * world";
  if ((reinterpret_cast<uintptr_t>(mc) & 15) || (reinterpret_cast<uintptr_t>(local) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return "nvls_all_reduce: buffers must be 16-byte aligned";
  PeerTable f = flags;
  uint4* mcp = static_cast<uint4*>(mc);
  const uint4* lp = static_cast<const uint4*>(local);
  uint4* op = static_cast<uint4*>(out);
  long long n16 = nbytes / 16;
  uint32_t ep = epoch;
  uint64_t lim = limit_ns;
  void* args[] = {&mcp, &lp, &f, &op, &n16, &rank, &world, &ep, &lim, &status, &abort_word};
  void* fn = dtype == kF32 ? reinterpret_cast<void*>(nvls_all_reduce_kernel<float>)
                           : reinterpret_cast<void*>(nvls_all_reduce_kernel<__nv_bfloat16>);
  // a small grid: the switch does the arithmetic, the SMs only issue 16-byte requests
  long long want = (n16 + 2047) / 2048;
  int grid = static_cast<int>(want < 1 ? 1 : (want > num_sms ? num_sms : want));
  if (cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(512), args, 0, s) != cudaSuccess)
    return "nvls_all_reduce: cooperative launch failed";
  count_launch();
  return nullptr;
}

}  // namespace ferrl
