// Expert-parallel dispatch and combine over NVLink peer memory.
//
// The reference replicates every expert on every rank (crates/ferrl/src/moe.rs:122-157); sharding
// the experts over ranks is added here.  Rank d owns the global experts [d*El, (d+1)*El).  Both
// directions of the all-to-all are single cooperative kernels working on a symmetric heap:
//
//   ep_dispatch_kernel   exchange per-expert counts (peer stores + bounded barrier); plan: every
//                        rank derives, from the same count matrix, the row each of its (token, slot)
//                        pairs takes in the owner's buffer (experts in 128-row aligned segments,
//                        source ranks in rank order inside a segment, pairs in stable order);
//                        push the token rows straight into the owners' buffers; barrier.
//   ep_combine_kernel    barrier (all experts' outputs are complete), then every rank pulls the
//                        rows of its own pairs from the owners and forms the weighted sum per token
//                        in slot order (deterministic), optionally keeping the pulled rows for the
//                        routing-weight gradient.
//
// The local experts then run the grouped tcgen05 GEMM over the received segments unchanged.  All
// peer waits are bounded and report through the status word; an over-full receive buffer is
// detected identically on every rank from the shared count matrix and reported the same way.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"
#include "../symm/symm.cuh"

namespace cg = cooperative_groups;

namespace ferrl {
namespace {

constexpr int kSeg = 128;
// The flag buffer belongs to the expert-parallel runtime alone: three barrier slots, then the call number.  The
// number lives on the device and each kernel advances it when it is through with its barriers, so a captured CUDA
// graph (the decode step) replays with fresh flag values; ranks call in lockstep, so their numbers agree.
constexpr int kSlotCounts = 0, kSlotPushed = 1, kSlotExperts = 2, kCallWord = 3 * kMaxRanks;
__device__ __forceinline__ volatile uint32_t* ep_call_word(const PeerTable& flags, int rank) {
  return static_cast<volatile uint32_t*>(flags.ptr[rank]) + kCallWord;
}

__device__ __forceinline__ int pad_seg(int n) { return (n + kSeg - 1) / kSeg * kSeg; }

__global__ void __launch_bounds__(512) ep_dispatch_kernel(EpDispatchParams p) {
  cg::grid_group grid = cg::this_grid();
  __shared__ int s_base, s_off, s_running, s_warp[16];
  volatile int* abort_word = p.abort_word;
  const int n_pairs = p.T * p.k;
  uint32_t epoch = 0;                              // used by thread 0 of block 0 only
  if (blockIdx.x == 0 && threadIdx.x == 0) epoch = *ep_call_word(p.flags, p.rank) + 1;

  if (!p.reuse_plan) {
    // ---- phase 0: publish my per-expert counts to every rank, wait for everyone's
    if (blockIdx.x == 0) {
      for (int d = 0; d < p.world; ++d) {
        int* dst = static_cast<int*>(p.counts_all.ptr[d]) + p.rank * p.E;
        for (int e = threadIdx.x; e < p.E; e += blockDim.x) dst[e] = p.my_counts[e];
      }
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) {
        const bool ok = peer_barrier(p.flags, kSlotCounts, p.rank, p.world, epoch, p.limit_ns, p.status);
        *abort_word = ok ? 0 : 1;
        __threadfence();
      }
    }
    grid.sync();
    if (*abort_word) return;

    // ---- phase 1: plan.  One block per global expert at a time.
    const int* all = static_cast<const int*>(p.counts_all.ptr[p.rank]);
    for (int e = blockIdx.x; e < p.E; e += gridDim.x) {
      const int owner = e / p.E_local;
      if (threadIdx.x == 0) {
        int base = 0;
        for (int e2 = owner * p.E_local; e2 < e; ++e2) {
          int tot = 0;
          for (int r = 0; r < p.world; ++r) tot += all[r * p.E + e2];
          base += pad_seg(tot);
        }
        int tot = 0, off = 0;
        for (int r = 0; r < p.world; ++r) {
          if (r < p.rank) off += all[r * p.E + e];
          tot += all[r * p.E + e];
        }
        s_base = base;
        s_off = off;
        s_running = 0;
        const int end = base + pad_seg(tot);
        if (end > p.cap_rows) {
          atomicCAS(p.status, kStatusOk, kStatusBadShape);   // same verdict on every rank
          *abort_word = 1;
        } else if (owner == p.rank) {
          for (int t = base / kSeg; t < end / kSeg; ++t) p.tile_expert[t] = e - owner * p.E_local;
          if (e == (owner + 1) * p.E_local - 1) {
            for (int t = end / kSeg; t < p.cap_rows / kSeg; ++t) p.tile_expert[t] = -1;
            *p.local_rows = end;
          }
        }
      }
      __syncthreads();
      const int first = s_base + s_off;
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
      for (int start = 0; start < n_pairs; start += blockDim.x) {
        const int i = start + threadIdx.x;
        const bool hit = i < n_pairs && p.idx[i] == e;
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) s_warp[warp] = __popc(ballot);
        __syncthreads();
        int before = s_running;
        for (int w = 0; w < warp; ++w) before += s_warp[w];
        if (hit) p.dest_row[i] = first + before + __popc(ballot & ((1u << lane) - 1));
        __syncthreads();
        if (threadIdx.x == 0) {
          int tot = 0;
          for (int w = 0; w < nwarps; ++w) tot += s_warp[w];
          s_running += tot;
        }
        __syncthreads();
      }
    }
    __threadfence();
    grid.sync();
    if (*abort_word) return;
  }

  // ---- phase 2: push rows into the owners' buffers (16-byte stores, coalesced along the row)
  const int chunks = p.H / 8;
  const long long n = static_cast<long long>(n_pairs) * chunks;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pair = static_cast<int>(i / chunks), c = static_cast<int>(i % chunks);
    uint4 v = *reinterpret_cast<const uint4*>(p.x + static_cast<long long>(pair / p.k) * p.ldx + c * 8);
    if (p.pair_w) {
      const float s = p.pair_w[pair];
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 f = __bfloat1622float2(h[q]);
        h[q] = __floats2bfloat162_rn(f.x * s, f.y * s);
      }
    }
    const int owner = p.idx[pair] / p.E_local;
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.xs.ptr[owner]) + static_cast<long long>(p.dest_row[pair]) * p.H;
    *reinterpret_cast<uint4*>(dst + c * 8) = v;
  }
  __threadfence_system();
  grid.sync();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const bool ok = peer_barrier(p.flags, kSlotPushed, p.rank, p.world, epoch, p.limit_ns, p.status);
    if (!ok) *abort_word = 1;
    *ep_call_word(p.flags, p.rank) = epoch;
  }
}

__global__ void __launch_bounds__(512) ep_combine_kernel(EpCombineParams p) {
  cg::grid_group grid = cg::this_grid();
  volatile int* abort_word = p.abort_word;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const uint32_t epoch = *ep_call_word(p.flags, p.rank) + 1;
    const bool ok = peer_barrier(p.flags, kSlotExperts, p.rank, p.world, epoch, p.limit_ns, p.status);
    *abort_word = ok ? 0 : 1;
    *ep_call_word(p.flags, p.rank) = epoch;
    __threadfence();
  }
  grid.sync();
  if (*abort_word) return;
  const int chunks = p.H / 8;
  const long long n = static_cast<long long>(p.T) * chunks;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / chunks), c = static_cast<int>(i % chunks);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < p.k; ++j) {
      const int pair = t * p.k + j;
      const int owner = p.idx[pair] / p.E_local;
      const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.ys.ptr[owner]) +
                                                      static_cast<long long>(p.dest_row[pair]) * p.H + c * 8);
      if (p.keep_rows) *reinterpret_cast<uint4*>(p.keep_rows + static_cast<long long>(pair) * p.H + c * 8) = v;
      const float s = p.w ? p.w[pair] : 1.f;
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += s * f.x;
        acc[2 * q + 1] += s * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    *reinterpret_cast<uint4*>(p.out + static_cast<long long>(t) * p.H + c * 8) = o;
  }
}

}  // namespace

const char* ep_dispatch(const EpDispatchParams& params, int num_sms, cudaStream_t stream) {
  if (params.H % 8) return "ep_dispatch: H % 8";
  if (params.world < 1 || params.world > kMaxRanks || params.E % params.world || params.E_local * params.world != params.E)
    return "ep_dispatch: experts must split evenly over ranks";
  if (params.cap_rows % kSeg) return "ep_dispatch: capacity must be a multiple of 128 rows";
  EpDispatchParams p = params;
  void* args[] = {&p};
  if (cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ep_dispatch_kernel), dim3(num_sms), dim3(512), args, 0, stream) !=
      cudaSuccess)
    return "ep_dispatch: cooperative launch failed";
  count_launch();
  return nullptr;
}

const char* ep_combine(const EpCombineParams& params, int num_sms, cudaStream_t stream) {
  if (params.H % 8) return "ep_combine: H % 8";
  EpCombineParams p = params;
  void* args[] = {&p};
  if (cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ep_combine_kernel), dim3(num_sms), dim3(512), args, 0, stream) !=
      cudaSuccess)
    return "ep_combine: cooperative launch failed";
  count_launch();
  return nullptr;
}

}  // namespace ferrl
