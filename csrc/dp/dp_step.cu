// Data-parallel LoRA step in ONE cooperative kernel over NVLink peer memory:
//
//   cross-rank barrier -> reduce-scatter of the flat gradient buffer (each rank sums its slice
//   over all peers with plain peer loads, in rank order, applies the 1/(accum*world) scale and
//   accumulates sum g^2) -> cross-rank barrier -> every rank combines the per-rank partial
//   norms (same order everywhere => identical bits) -> global-norm clip factor -> AdamW on the
//   fp32 master adapters, reading each reduced slice from its owner (the all-gather half of the
//   all-reduce is folded into the optimizer's read).
//
// The reference issues one blocking ncclAllReduce per gradient tensor in chunks of 16, then a
// host-synchronised f64 norm per tensor, then ~10 elementwise launches per tensor for Adam.
//
// Rank order is fixed, partial norms are combined by one block in index order, and nothing uses
// floating-point atomics, so ranks stay in bitwise lockstep and reruns are bit-reproducible.
// Non-finite reduced gradients and host-reported uncovered tensors are counted world-wide; if
// any exist, or the global norm is exactly zero, no rank updates anything.
// Both peer waits are bounded (see symm.cuh); on expiry the kernel reports and returns.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"
#include "../symm/symm.cuh"

namespace cg = cooperative_groups;

namespace ferrl {
namespace {

__global__ void __launch_bounds__(512) dp_step_kernel(DpStepParams p) {
  cg::grid_group grid = cg::this_grid();
  __shared__ float red[32];
  __shared__ double dred[32];
  int* abort_word = p.abort_word;

  // ---- barrier A: every rank's gradients are complete in its symmetric buffer
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    bool ok = peer_barrier(p.flags, 0, p.rank, p.barrier_world, p.epoch, p.limit_ns, p.status);
    *abort_word = ok ? 0 : 1;
    __threadfence();
  }
  grid.sync();
  if (*reinterpret_cast<volatile int*>(abort_word)) return;

  // ---- phase 1: reduce my slice(s), scale, sum of squares, non-finite count
  const long long slice = p.n / p.world;  // n is padded to a multiple of 4*world
  float ss = 0.f, bad = 0.f;
  for (int owner = p.own_lo; owner < p.own_hi; ++owner) {
    const long long base = static_cast<long long>(owner) * slice;
    float* dst = static_cast<float*>(p.reduced.ptr[owner]) + base;
    const long long n4 = slice / 4;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int q = 0; q < p.world; ++q) {
        const float4 v = reinterpret_cast<const float4*>(static_cast<const float*>(p.grads.ptr[q]) + base)[i];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      acc.x *= p.pre_scale; acc.y *= p.pre_scale; acc.z *= p.pre_scale; acc.w *= p.pre_scale;
      reinterpret_cast<float4*>(dst)[i] = acc;
      ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
      if (!isfinite(acc.x) || !isfinite(acc.y) || !isfinite(acc.z) || !isfinite(acc.w)) bad += 1.f;
    }
  }
  float tot = block_sum(ss, red);
  float nb = block_sum(bad, red);
  if (threadIdx.x == 0) {
    p.block_partials[2 * blockIdx.x] = static_cast<double>(tot);
    p.block_partials[2 * blockIdx.x + 1] = static_cast<double>(nb);
  }
  __threadfence();
  grid.sync();

  // ---- block 0 folds the per-block partials in index order, publishes, barrier B
  if (blockIdx.x == 0) {
    double s = 0.0, b = 0.0;
    for (int i = threadIdx.x; i < static_cast<int>(gridDim.x); i += blockDim.x) {
      // strided partial sums are then combined in lane order below: still a fixed order
      s += p.block_partials[2 * i];
      b += p.block_partials[2 * i + 1];
    }
    // deterministic tree: warp shuffles then one thread walks the warp totals
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    if ((threadIdx.x & 31) == 0) {
      dred[threadIdx.x >> 5] = s;
      dred[16 + (threadIdx.x >> 5)] = b;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      double S = 0.0, B = 0.0;
      for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) {
        S += dred[w];
        B += dred[16 + w];
      }
      double* mine = static_cast<double*>(p.scalars.ptr[p.rank]);
      mine[0] = S;
      mine[1] = B + static_cast<double>(p.uncovered_local);
      bool ok = peer_barrier(p.flags, 1, p.rank, p.barrier_world, p.epoch, p.limit_ns, p.status);
      *abort_word = ok ? 0 : 1;
      __threadfence();
    }
  }
  grid.sync();
  if (*reinterpret_cast<volatile int*>(abort_word)) return;

  // ---- phase 2: global norm (same order on every rank), clip, AdamW reading reduced slices from owners
  double total = 0.0, unc = 0.0;
  for (int q = 0; q < p.world; ++q) {
    const double* sc = static_cast<const double*>(p.scalars.ptr[q]);
    total += sc[0];
    unc += sc[1];
  }
  const float norm = static_cast<float>(sqrt(total));
  const bool step = (unc == 0.0) && (norm > 0.f) && isfinite(norm);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    p.out[0] = norm;
    p.out[1] = static_cast<float>(unc);
    p.out[2] = step ? 1.f : 0.f;
  }
  if (!step) return;
  float gs = 1.f;
  if (p.max_norm > 0.f && norm > p.max_norm) gs = p.max_norm / norm;
  for (int blk = blockIdx.x; blk < p.n_blocks; blk += gridDim.x) {
    const AdamTensor t = p.tab[p.blk_tensor[blk]];
    const long long off = p.blk_off[blk];
    const long long end = min(off + static_cast<long long>(p.chunk), t.n);
    const long long flat0 = p.blk_flat[blk];
    for (long long i = off + threadIdx.x; i < end; i += blockDim.x) {
      const long long f = flat0 + (i - off);
      const int owner = static_cast<int>(f / slice);
      float g = static_cast<const float*>(p.reduced.ptr[owner])[f] * gs;
      float m = p.b1 * t.m[i] + (1.f - p.b1) * g;
      float v = p.b2 * t.v[i] + (1.f - p.b2) * g * g;
      float w = t.p[i] * (1.f - p.lr * p.wd);
      w -= p.lr * (m * p.bc1_inv) / (sqrtf(v * p.bc2_inv) + p.eps);
      t.m[i] = m;
      t.v[i] = v;
      t.p[i] = w;
    }
  }
}

// Sum all-reduce of a symmetric buffer (bf16 or fp32), used for tensor-parallel activations.  Deterministic and
// identical on every rank (every element is summed once, in rank order, by one rank).
//   world <= 2  one shot: barrier, every rank reads all peers' copies of the whole range, barrier;
//   world  > 2  two shots: rank r sums slice r of all copies and stores the result into slice r of EVERY copy
//               (in place: nobody else reads slice r), barrier, every rank copies its now complete local buffer
//               out.  Per rank 2 (world-1)/world n elements cross NVLink instead of (world-1) n.
template <typename T>
__global__ void __launch_bounds__(512) symm_all_reduce_kernel(PeerTable src, PeerTable flags, T* __restrict__ out,
                                                             long long n, int rank, int world, uint32_t epoch,
                                                             uint64_t limit_ns, int* status, int* abort_word) {
  cg::grid_group grid = cg::this_grid();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    bool ok = peer_barrier(flags, 2, rank, world, epoch, limit_ns, status);
    *abort_word = ok ? 0 : 1;
    __threadfence();
  }
  grid.sync();
  if (*reinterpret_cast<volatile int*>(abort_word)) return;
  constexpr int VEC = 16 / sizeof(T);
  const long long nv = n / VEC;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const bool two_shot = world > 2;
  // the 16-byte units this rank sums: everything (one shot) or its slice (two shots; the last rank takes the remainder)
  const long long per = two_shot ? nv / world : nv;
  const long long lo = two_shot ? per * rank : 0;
  const long long hi = two_shot ? (rank == world - 1 ? nv : lo + per) : nv;
  for (long long i = lo + tid; i < hi; i += nthreads) {
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    for (int q = 0; q < world; ++q) {
      uint4 raw = reinterpret_cast<const uint4*>(src.ptr[q])[i];
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] += to_f(v[e]);
    }
    uint4 o;
    T* ov = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int e = 0; e < VEC; ++e) ov[e] = from_f<T>(acc[e]);
    if (two_shot) {
      for (int q = 0; q < world; ++q) reinterpret_cast<uint4*>(src.ptr[q])[i] = o;
    } else {
      reinterpret_cast<uint4*>(out)[i] = o;
    }
  }
  // the tail that does not fill a 16-byte unit: rank 0's job in the two-shot form
  if (!two_shot || rank == 0) {
    for (long long i = nv * VEC + tid; i < n; i += nthreads) {
      float acc = 0.f;
      for (int q = 0; q < world; ++q) acc += to_f(static_cast<const T*>(src.ptr[q])[i]);
      if (two_shot) {
        for (int q = 0; q < world; ++q) static_cast<T*>(src.ptr[q])[i] = from_f<T>(acc);
      } else {
        out[i] = from_f<T>(acc);
      }
    }
  }
  grid.sync();
  // trailing barrier: one shot - nobody may overwrite its source buffer until every peer has read it;
  // two shots - every slice has been reduced and stored into this rank's copy
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    bool ok = peer_barrier(flags, 3, rank, world, epoch, limit_ns, status);
    if (!ok) *abort_word = 1;
    __threadfence();
  }
  if (!two_shot) return;
  grid.sync();
  if (*reinterpret_cast<volatile int*>(abort_word)) return;
  const T* mine = static_cast<const T*>(src.ptr[rank]);
  for (long long i = tid; i < nv; i += nthreads) reinterpret_cast<uint4*>(out)[i] = reinterpret_cast<const uint4*>(mine)[i];
  for (long long i = nv * VEC + tid; i < n; i += nthreads) out[i] = mine[i];
}

// The two halves of the all-reduce as collectives of their own, for sequence-sharded tensor parallelism (the
// residual stream holds 1 / world of the token rows between a row-parallel projection and the next column-parallel
// one).  Rows are contiguous, so a shard is a contiguous range of n_shard elements.
//   reduce-scatter: src[q] holds rank q's full partial [world * n_shard]; rank r sums slice r over q (rank order)
//                   into `out` [n_shard].  Leading barrier: all partials staged; trailing: all slices read.
//   all-gather:     src[q] holds rank q's shard [n_shard]; every rank copies all shards into `out` [world * n_shard].
template <typename T>
__global__ void __launch_bounds__(512) symm_reduce_scatter_kernel(PeerTable src, PeerTable flags, T* __restrict__ out,
                                                                 long long n_shard, int rank, int world, uint32_t epoch,
                                                                 uint64_t limit_ns, int* status, int* abort_word) {
  cg::grid_group grid = cg::this_grid();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    bool ok = peer_barrier(flags, 6, rank, world, epoch, limit_ns, status);
    *abort_word = ok ? 0 : 1;
    __threadfence();
  }
  grid.sync();
  if (*reinterpret_cast<volatile int*>(abort_word)) return;
  constexpr int VEC = 16 / sizeof(T);
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long base = n_shard * rank;                       // first element of this rank's slice in every partial
  const bool vec = (n_shard % VEC) == 0;                       // then every slice starts on a 16-byte boundary
  const long long nv = vec ? n_shard / VEC : 0;
  for (long long i = tid; i < nv; i += nthreads) {
    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
    for (int q = 0; q < world; ++q) {
      uint4 raw = reinterpret_cast<const uint4*>(static_cast<const T*>(src.ptr[q]) + base)[i];
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] += to_f(v[e]);
    }
    uint4 o;
    T* ov = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int e = 0; e < VEC; ++e) ov[e] = from_f<T>(acc[e]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
  for (long long i = nv * VEC + tid; i < n_shard; i += nthreads) {
    float acc = 0.f;
    for (int q = 0; q < world; ++q) acc += to_f(static_cast<const T*>(src.ptr[q])[base + i]);
    out[i] = from_f<T>(acc);
  }
  grid.sync();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    bool ok = peer_barrier(flags, 7, rank, world, epoch, limit_ns, status);
    if (!ok) *abort_word = 1;
  }
}

template <typename T>
__global__ void __launch_bounds__(512) symm_all_gather_kernel(PeerTable src, PeerTable flags, T* __restrict__ out,
                                                             long long n_shard, int rank, int world, uint32_t epoch,
                                                             uint64_t limit_ns, int* status, int* abort_word) {
  cg::grid_group grid = cg::this_grid();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    bool ok = peer_barrier(flags, 6, rank, world, epoch, limit_ns, status);
    *abort_word = ok ? 0 : 1;
    __threadfence();
  }
  grid.sync();
  if (*reinterpret_cast<volatile int*>(abort_word)) return;
  constexpr int VEC = 16 / sizeof(T);
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const bool vec = (n_shard % VEC) == 0;
  const long long nv = vec ? n_shard / VEC : 0;
  for (int q = 0; q < world; ++q) {
    const T* from = static_cast<const T*>(src.ptr[q]);
    T* to = out + n_shard * q;
    for (long long i = tid; i < nv; i += nthreads) reinterpret_cast<uint4*>(to)[i] = reinterpret_cast<const uint4*>(from)[i];
    for (long long i = nv * VEC + tid; i < n_shard; i += nthreads) to[i] = from[i];
  }
  grid.sync();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    bool ok = peer_barrier(flags, 7, rank, world, epoch, limit_ns, status);
    if (!ok) *abort_word = 1;
  }
}

}  // namespace

const char* dp_step(const DpStepParams& p, int num_sms, cudaStream_t s) {
  if (p.world < 1 || p.world > kMaxRanks) return "dp_step: world size out of range";
  if (p.n % (4LL * p.world)) return "dp_step: flat length must be padded to a multiple of 4*world";
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dp_step_kernel, 512, 0) != cudaSuccess || per_sm < 1)
    return "dp_step: occupancy query failed";
  int grid = num_sms;  // one resident block per SM: cooperative launch needs co-residency
  DpStepParams q = p;
  void* args[] = {&q};
  if (cudaLaunchCooperativeKernel(reinterpret_cast<void*>(dp_step_kernel), dim3(grid), dim3(512), args, 0, s) !=
      cudaSuccess)
    return "dp_step: cooperative launch failed";
  count_launch();
  return nullptr;
}

int dp_step_grid(int num_sms) { return num_sms; }

const char* symm_all_reduce(int dtype, const PeerTable& src, const PeerTable& flags, void* out, long long n, int rank,
                            int world, unsigned epoch, unsigned long long limit_ns, int* status, int* abort_word,
                            int num_sms, cudaStream_t s) {
  if (world < 1 || world > kMaxRanks) return "symm_all_reduce: world size out of range";
  PeerTable a = src, f = flags;
  uint32_t ep = epoch;
  uint64_t lim = limit_ns;
  int grid = num_sms;
  void* args[] = {&a, &f, &out, &n, &rank, &world, &ep, &lim, &status, &abort_word};
  void* fn = dtype == kF32 ? reinterpret_cast<void*>(symm_all_reduce_kernel<float>)
                           : reinterpret_cast<void*>(symm_all_reduce_kernel<__nv_bfloat16>);
  if (cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(512), args, 0, s) != cudaSuccess)
    return "symm_all_reduce: cooperative launch failed";
  count_launch();
  return nullptr;
}

// which: 0 reduce-scatter (src = full partials, out = this rank's slice), 1 all-gather (src = shards, out = all rows)
const char* symm_row_collective(int which, int dtype, const PeerTable& src, const PeerTable& flags, void* out, long long n_shard,
                                int rank, int world, unsigned epoch, unsigned long long limit_ns, int* status, int* abort_word,
                                int num_sms, cudaStream_t s) {
  if (world < 1 || world > kMaxRanks) return "symm_row_collective: world size out of range";
  if (n_shard == 0) return nullptr;
  if ((n_shard * (dtype == kF32 ? 4 : 2)) % 16 == 0 && (reinterpret_cast<uintptr_t>(out) & 15)) return "symm_row_collective: output must be 16-byte aligned";
  PeerTable a = src, f = flags;
  uint32_t ep = epoch;
  uint64_t lim = limit_ns;
  void* args[] = {&a, &f, &out, &n_shard, &rank, &world, &ep, &lim, &status, &abort_word};
  void* fn;
  if (which == 0)
    fn = dtype == kF32 ? reinterpret_cast<void*>(symm_reduce_scatter_kernel<float>) : reinterpret_cast<void*>(symm_reduce_scatter_kernel<__nv_bfloat16>);
  else
    fn = dtype == kF32 ? reinterpret_cast<void*>(symm_all_gather_kernel<float>) : reinterpret_cast<void*>(symm_all_gather_kernel<__nv_bfloat16>);
  if (cudaLaunchCooperativeKernel(fn, dim3(num_sms), dim3(512), args, 0, s) != cudaSuccess)
    return "symm_row_collective: cooperative launch failed";
  count_launch();
  return nullptr;
}

}  // namespace ferrl
