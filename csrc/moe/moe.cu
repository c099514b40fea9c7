// Mixture-of-experts routing, dispatch and combine for sm_100a.
//
// The reference loops over experts on the host and copies the routing table to the host once
// per layer (crates/ferrl/src/moe.rs:110-158).  Here the whole plan stays on the device:
//
//   moe_route_kernel    softmax over E router logits (fp32), top-k, renormalise, count rows/expert
//   moe_plan_kernel     stable counting sort of the T*k (token, slot) pairs by expert into
//                       128-row aligned segments: row_of[pair], token_of[row], tile_expert[m tile]
//   moe_gather_kernel   xs[row] = scale(row) * x[token_of[row]]   (zero rows for padding)
//   (grouped tcgen05 GEMM over the segments: csrc/gemm/tcgen05_gemm.cu, tile_expert mode)
//   moe_combine_kernel  out[t] = sum_j w[t,j] * ys[row_of[t,j]]   (fixed order, fp32 accumulate)
//   moe_pair_dot_kernel dw[t,j] = <dy[t], ys[row_of[t,j]]>        (router-weight gradient)
//
// The padded layout makes every 128-row m tile belong to exactly one expert, so the grouped GEMM
// is the ordinary persistent kernel with one extra table lookup per tile; no host sync anywhere.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "../api.h"
#include "../common.cuh"

namespace ferrl {

namespace {

constexpr int kMaxTopK = 16;
constexpr int kSeg = 128;   // segment alignment = GEMM tile height

// One warp per token. logits [T, E] fp32 (row stride ld); E <= 1024.
__global__ void moe_route_kernel(const float* __restrict__ logits, long long ld, int T, int E, int k, int renorm,
                                 float* __restrict__ probs, float* __restrict__ scores, int* __restrict__ idx,
                                 int* __restrict__ counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + static_cast<long long>(warp) * ld;
  float v[32];   // up to 1024 experts, 32 per lane
  const int per = (E + 31) / 32;
  float mx = -INFINITY;
  for (int i = 0; i < per; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
  for (int i = 0; i < per; ++i) {
    v[i] = (i * 32 + lane < E) ? __expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  for (int i = 0; i < per; ++i) {
    v[i] *= inv;
    const int e = i * 32 + lane;
    if (probs && e < E) probs[static_cast<long long>(warp) * E + e] = v[i];
  }
  // k rounds of arg-max; ties go to the lower expert index (matches a stable descending sort)
  float top_sum = 0.f;
  float my_score = 0.f;
  int my_idx = 0;
  for (int j = 0; j < k; ++j) {
    float best = -1.f;
    int best_e = 0x7fffffff;
    for (int i = 0; i < per; ++i) {
      const int e = i * 32 + lane;
      if (e < E && v[i] > best) {
        best = v[i];
        best_e = e;
      }
    }
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if ((best_e & 31) == lane) v[best_e >> 5] = -2.f;   // taken
    top_sum += best;
    if (lane == j) {
      my_score = best;
      my_idx = best_e;
    }
  }
  if (lane < k) {
    scores[static_cast<long long>(warp) * k + lane] = renorm ? my_score / top_sum : my_score;
    idx[static_cast<long long>(warp) * k + lane] = my_idx;
    atomicAdd(&counts[my_idx], 1);   // integer counts: order-independent
  }
}

// One block per expert: stable rank of every pair routed to this expert.
__global__ void moe_plan_kernel(const int* __restrict__ idx, const int* __restrict__ counts, int n_pairs, int k, int E,
                                int max_rows, int* __restrict__ row_of, int* __restrict__ token_of,
                                int* __restrict__ tile_expert, int* __restrict__ seg_start) {
  const int e = blockIdx.x;
  __shared__ int s_base, s_warp[32], s_running;
  if (threadIdx.x == 0) {
    int base = 0;
    for (int i = 0; i < e; ++i) base += (counts[i] + kSeg - 1) / kSeg * kSeg;
    s_base = base;
    s_running = 0;
    if (seg_start) seg_start[e] = base;
    if (e == E - 1) {
      // tiles past the last segment stay unused
      const int end = base + (counts[e] + kSeg - 1) / kSeg * kSeg;
      if (seg_start) seg_start[E] = end;
      for (int t = end / kSeg; t < max_rows / kSeg; ++t) tile_expert[t] = -1;
    }
  }
  __syncthreads();
  const int base = s_base;
  const int cnt = counts[e];
  const int padded = (cnt + kSeg - 1) / kSeg * kSeg;
  for (int t = threadIdx.x; t < padded / kSeg; t += blockDim.x) tile_expert[base / kSeg + t] = e;
  for (int r = cnt + threadIdx.x; r < padded; r += blockDim.x) token_of[base + r] = -1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int start = 0; start < n_pairs; start += blockDim.x) {
    const int i = start + threadIdx.x;
    const bool hit = i < n_pairs && idx[i] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    int before = s_running;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    if (hit) {
      const int r = base + before + __popc(ballot & ((1u << lane) - 1));
      row_of[i] = r;
      token_of[r] = i / k;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < nwarps; ++w) tot += s_warp[w];
      s_running += tot;
    }
    __syncthreads();
  }
}

// xs[row, :] = (w ? w[pair_of_row] : 1) * x[token_of[row], :]; H % 8 == 0.  pair scale is looked up
// through row_of's inverse, passed as `row_scale` [rows] (or null).
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ token_of,
                                  const float* __restrict__ row_scale, int rows, int H,
                                  __nv_bfloat16* __restrict__ xs) {
  const int chunks = H / 8;
  const long long n = static_cast<long long>(rows) * chunks;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / chunks), c = static_cast<int>(i % chunks);
    const int t = token_of[r];
    uint4 o = make_uint4(0, 0, 0, 0);
    if (t >= 0) {
      o = *reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * ldx + c * 8);
      if (row_scale) {
        const float s = row_scale[r];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = __bfloat1622float2(h[e]);
          h[e] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
      }
    }
    *reinterpret_cast<uint4*>(xs + static_cast<long long>(r) * H + c * 8) = o;
  }
}

// row_scale[row_of[pair]] = w[pair]
__global__ void moe_row_scale_kernel(const float* __restrict__ w, const int* __restrict__ row_of, int n_pairs,
                                     float* __restrict__ row_scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_pairs) row_scale[row_of[i]] = w[i];
}

// out[t, :] = sum_j w[t, j] * ys[row_of[t*k + j], :]   (w null -> plain sum)
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ row_of,
                                   const float* __restrict__ w, int T, int k, int H, __nv_bfloat16* __restrict__ out) {
  const int chunks = H / 8;
  const long long n = static_cast<long long>(T) * chunks;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / chunks), c = static_cast<int>(i % chunks);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int r = row_of[static_cast<long long>(t) * k + j];
      const float s = w ? w[static_cast<long long>(t) * k + j] : 1.f;
      const uint4 v = *reinterpret_cast<const uint4*>(ys + static_cast<long long>(r) * H + c * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += s * f.x;
        acc[2 * e + 1] += s * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * H + c * 8) = o;
  }
}

// dw[pair] = <dy[pair / k, :], ys[row_of[pair], :]>, one warp per pair
__global__ void moe_pair_dot_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ ys,
                                    const int* __restrict__ row_of, int n_pairs, int k, int H, float* __restrict__ dw) {
  const int pair = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (pair >= n_pairs) return;
  const __nv_bfloat16* a = dy + static_cast<long long>(pair / k) * H;
  const __nv_bfloat16* b = ys + static_cast<long long>(row_of[pair]) * H;
  float acc = 0.f;
  for (int c = lane; c < H / 8; c += 32) {
    const uint4 va = *reinterpret_cast<const uint4*>(a + c * 8);
    const uint4 vb = *reinterpret_cast<const uint4*>(b + c * 8);
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&va);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&vb);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 fa = __bfloat1622float2(ha[e]), fb = __bfloat1622float2(hb[e]);
      acc += fa.x * fb.x + fa.y * fb.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) dw[pair] = acc;
}

}  // namespace

const char* moe_route(const float* logits, long long ld, int T, int E, int k, bool renorm, float* probs, float* scores,
                      int* idx, int* counts, cudaStream_t stream) {
  if (E > 1024 || k > kMaxTopK || k > E || k > 32) return "moe_route: E <= 1024 and k <= 16 supported";
  if (T == 0) return nullptr;
  cudaMemsetAsync(counts, 0, sizeof(int) * E, stream);
  const int threads = 256, warps = threads / 32;
  moe_route_kernel<<<(T + warps - 1) / warps, threads, 0, stream>>>(logits, ld, T, E, k, renorm ? 1 : 0, probs, scores,
                                                                   idx, counts);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "moe_route launch failed";
}

const char* moe_plan(const int* idx, const int* counts, int n_pairs, int k, int E, int max_rows, int* row_of,
                     int* token_of, int* tile_expert, int* seg_start, cudaStream_t stream) {
  if (max_rows % kSeg) return "moe_plan: max_rows must be a multiple of 128";
  moe_plan_kernel<<<E, 1024, 0, stream>>>(idx, counts, n_pairs, k, E, max_rows, row_of, token_of, tile_expert, seg_start);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "moe_plan launch failed";
}

const char* moe_gather(const void* x, long long ldx, const int* token_of, const float* pair_w, const int* row_of,
                       int n_pairs, float* row_scale, int rows, int H, void* xs, cudaStream_t stream) {
  if (H % 8) return "moe_gather: H % 8";
  if (pair_w) {
    moe_row_scale_kernel<<<(n_pairs + 255) / 256, 256, 0, stream>>>(pair_w, row_of, n_pairs, row_scale);
    count_launch();
  }
  const long long n = static_cast<long long>(rows) * (H / 8);
  const int blocks = static_cast<int>(std::min<long long>((n + 255) / 256, 148 * 16));
  moe_gather_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ldx, token_of,
                                                pair_w ? row_scale : nullptr, rows, H, static_cast<__nv_bfloat16*>(xs));
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "moe_gather launch failed";
}

const char* moe_combine(const void* ys, const int* row_of, const float* w, int T, int k, int H, void* out,
                        cudaStream_t stream) {
  if (H % 8) return "moe_combine: H % 8";
  if (T == 0) return nullptr;
  const long long n = static_cast<long long>(T) * (H / 8);
  const int blocks = static_cast<int>(std::min<long long>((n + 255) / 256, 148 * 16));
  moe_combine_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(ys), row_of, w, T, k, H,
                                                 static_cast<__nv_bfloat16*>(out));
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "moe_combine launch failed";
}

const char* moe_pair_dot(const void* dy, const void* ys, const int* row_of, int n_pairs, int k, int H, float* dw,
                         cudaStream_t stream) {
  if (H % 8) return "moe_pair_dot: H % 8";
  if (n_pairs == 0) return nullptr;
  const int threads = 256, warps = threads / 32;
  moe_pair_dot_kernel<<<(n_pairs + warps - 1) / warps, threads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(ys), row_of, n_pairs, k, H, dw);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "moe_pair_dot launch failed";
}

}  // namespace ferrl
