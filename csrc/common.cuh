// Shared device/host helpers for the sm_100a kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ferrl {

// Error codes written to a device status word instead of trapping. A kernel that
// gives up on a bounded wait records where and returns normally so the context
// stays usable; the host reads the word after the stream sync.
enum : int {
  kStatusOk = 0,
  kStatusWaitTimeoutProducer = 1,
  kStatusWaitTimeoutMma = 2,
  kStatusWaitTimeoutEpilogue = 3,
  kStatusPeerWaitTimeout = 4,
  kStatusBadShape = 5,
};

#ifdef __CUDACC__
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum over blockDim.x threads (multiple of 32, <= 1024). `red` is a
// shared float[32]. Result is returned to every thread.
__device__ __forceinline__ float block_sum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float r = (lane < nw) ? red[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Programmatic dependent launch.  A kernel launched with launch_pdl() may begin while its stream
// predecessor is still running, once every CTA of the predecessor has executed pdl_trigger() (or
// exited); it must execute pdl_wait() before it touches anything the predecessor writes, and before
// it writes anything the predecessor reads.  Both instructions are no-ops in an ordinary launch.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

#endif  // __CUDACC__

#ifdef __CUDACC__
// Launch `kern` so that it may overlap the tail of its stream predecessor (see pdl_wait()).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

// cudaFuncSetAttribute values are per device: a flag that remembers "already set" must be kept per
// device too, or a process that drives a second GPU launches there without the opt-in.  This is a
// once-per-(call site, device) guard; devices beyond kMaxDevices simply set the attribute every time.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
  unsigned char done[kMaxDevices] = {};   // written with the same value by any racing thread
  // Returns the current device's slot index, or -1 when it cannot be cached.
  static int slot() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
  }
};
// `expr` evaluates to true when every attribute call succeeded.  Evaluates to false on failure.
#define FERRL_ONCE_PER_DEVICE(expr)                                                         \
  ([&]() -> bool {                                                                          \
    static ::ferrl::PerDeviceOnce once_;                                                    \
    const int slot_ = ::ferrl::PerDeviceOnce::slot();                                       \
    if (slot_ >= 0 && once_.done[slot_]) return true;                                       \
    if (!(expr)) return false;                                                              \
    if (slot_ >= 0) once_.done[slot_] = 1;                                                  \
    return true;                                                                            \
  }())

// Count of kernel launches issued by this library (host side, for benchmarks).
void count_launch(int n = 1);
long long launch_count();

}  // namespace ferrl
