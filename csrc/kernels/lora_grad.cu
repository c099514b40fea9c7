// Adapter gradients: out[R, C] = U^T X with U [M, R] and X [M, C] bf16, fp32 result.
//
//   dA = (dy B)^T x        U = dy B  [tokens, R],  X = x   [tokens, K]
//   dB^T = t^T dy          U = x A^T [tokens, R],  X = dy  [tokens, N]
//
// The reduction runs over the token dimension, which is the strided one in both operands, so the
// TMA/tcgen05 GEMM (K-major operands) does not apply without materialising transposes of the
// activations.  Here both operands are streamed once, row-major, through a cp.async ring and the
// transposed fragments come out of ldmatrix.trans; the products run on mma.sync m16n8k16.
// Work is split over column tiles and token ranges; the per-range partial tiles are summed by the
// last CTA of each column tile in range order, so the result does not depend on scheduling.
// The reference forms these products with candle matmuls on transposed views
// (crates/ferrl/src/lora.rs backward of the adapter path).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "../api.h"
#include "../common.cuh"
#include "mma_sync.cuh"

namespace ferrl {
namespace {

using namespace mmah;

constexpr int LG_COLS = 128;     // output columns per CTA
constexpr int LG_ROWS = 64;      // tokens per stage
constexpr int LG_STAGES = 3;
constexpr int LG_TILE_BYTES = LG_ROWS * 256;   // both tiles use 256-byte rows (128 bf16)

template <int RT>   // RT 16-row tiles of R (R <= 16*RT <= 128)
__global__ void __launch_bounds__(128)
lora_grad_kernel(const __nv_bfloat16* __restrict__ U, long long ldu, int R, const __nv_bfloat16* __restrict__ X,
                 long long ldx, int C, int M, int rows_per_split, float* __restrict__ partial,
                 int* __restrict__ counters, float* __restrict__ out, long long ldo) {
  extern __shared__ __align__(128) uint8_t lsm[];
  __shared__ int s_last;
  const int ct = blockIdx.x, split = blockIdx.y, n_splits = gridDim.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = ct * LG_COLS;
  const int m_begin = split * rows_per_split, m_end = min(M, m_begin + rows_per_split);
  const int n_stages = m_end > m_begin ? (m_end - m_begin + LG_ROWS - 1) / LG_ROWS : 0;
  const int r_chunks = (R + 7) / 8;

  auto issue = [&](int s) {
    if (s < n_stages) {
      uint8_t* xt = lsm + (s % LG_STAGES) * 2 * LG_TILE_BYTES;
      uint8_t* ut = xt + LG_TILE_BYTES;
      const int m0 = m_begin + s * LG_ROWS;
      for (int i = threadIdx.x; i < LG_ROWS * 16; i += 128) {
        const int r = i >> 4, ch = i & 15;
        const bool ok = (m0 + r) < m_end && (c0 + ch * 8) < C;
        cp_async16(smem_addr(xt) + sw_off<256>(r, ch), X + static_cast<long long>(ok ? m0 + r : 0) * ldx + (ok ? c0 + ch * 8 : 0), ok);
      }
      for (int i = threadIdx.x; i < LG_ROWS * 2 * RT; i += 128) {
        const int r = i / (2 * RT), ch = i % (2 * RT);
        const bool ok = (m0 + r) < m_end && ch < r_chunks;
        cp_async16(smem_addr(ut) + sw_off<256>(r, ch), U + static_cast<long long>(ok ? m0 + r : 0) * ldu + (ok ? ch * 8 : 0), ok);
      }
    }
    cp_commit();
  };

  float acc[RT][4][4];
#pragma unroll
  for (int a = 0; a < RT; ++a)
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[a][n][e] = 0.f;

#pragma unroll
  for (int s = 0; s < LG_STAGES - 1; ++s) issue(s);
  for (int s = 0; s < n_stages; ++s) {
    cp_wait<LG_STAGES - 2>();
    __syncthreads();
    issue(s + LG_STAGES - 1);
    const uint8_t* xt = lsm + (s % LG_STAGES) * 2 * LG_TILE_BYTES;
    const uint8_t* ut = xt + LG_TILE_BYTES;
#pragma unroll
    for (int ks = 0; ks < LG_ROWS / 16; ++ks) {
      // B fragments: X[k = token][n = column], 4 n-tiles of this warp's 32 columns
      uint32_t b[8];
      {
        const int row = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int chunk = warp * 4 + (lane >> 4);
        ldsm4t(smem_addr(xt) + sw_off<256>(row, chunk), b[0], b[1], b[2], b[3]);
        ldsm4t(smem_addr(xt) + sw_off<256>(row, chunk + 2), b[4], b[5], b[6], b[7]);
      }
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        // A fragment: U^T[row = r][k = token] out of the [token][r] tile
        uint32_t a[4];
        const int mat = lane >> 3;
        const int row = ks * 16 + (lane & 7) + (mat >> 1) * 8;
        const int chunk = rt * 2 + (mat & 1);
        ldsm4t(smem_addr(ut) + sw_off<256>(row, chunk), a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int n = 0; n < 4; ++n) mma16816(acc[rt][n], a, b[2 * n], b[2 * n + 1]);
      }
    }
  }
  cp_wait<0>();

  // partial tile of this token range: [split][16*RT][C], fp32
  const int g = lane >> 2, t = lane & 3;
  float* part = partial + static_cast<long long>(split) * (16 * RT) * C;
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const int col = c0 + warp * 32 + n * 8 + 2 * t;
      if (col < C) {   // C % 8 == 0, so col + 1 < C as well
        *reinterpret_cast<float2*>(part + static_cast<long long>(rt * 16 + g) * C + col) = make_float2(acc[rt][n][0], acc[rt][n][1]);
        *reinterpret_cast<float2*>(part + static_cast<long long>(rt * 16 + g + 8) * C + col) = make_float2(acc[rt][n][2], acc[rt][n][3]);
      }
    }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int seen = atomicAdd(&counters[ct], 1);
    s_last = (seen == n_splits - 1);
    if (s_last) counters[ct] = 0;     // ready for the next call on this stream
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // the last CTA of this column tile sums the ranges in order
  for (int i = threadIdx.x; i < R * (LG_COLS / 4); i += 128) {
    const int r = i / (LG_COLS / 4), c = c0 + (i % (LG_COLS / 4)) * 4;
    if (c >= C) continue;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < n_splits; ++s) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(partial + (static_cast<long long>(s) * (16 * RT) + r) * C + c));
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    *reinterpret_cast<float4*>(out + static_cast<long long>(r) * ldo + c) = sum;
  }
}

}  // namespace

size_t lora_grad_workspace_floats(int R, int C, int n_splits) {
  const int rt = (R + 15) / 16;
  return static_cast<size_t>(n_splits) * rt * 16 * C;
}

int lora_grad_splits(int M, int C, int num_sms) {
  // Two CTAs fit on an SM.  The token split is chosen so that the grid fills whole waves of
  // 2 * num_sms CTAs: a grid of 1.08 waves takes as long as one of two.
  const int col_tiles = (C + LG_COLS - 1) / LG_COLS;
  const int slots = 2 * num_sms;
  const int max_s = std::min(64, std::max(1, (M + 4 * LG_ROWS - 1) / (4 * LG_ROWS)));   // at least four stages per CTA
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= max_s; ++s) {
    const long long ctas = static_cast<long long>(col_tiles) * s;
    const long long waves = (ctas + slots - 1) / slots;
    const double eff = static_cast<double>(ctas) / static_cast<double>(waves * slots);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = s;
    }
    if (eff >= 0.93 && ctas >= slots / 2) return s;      // smallest split that fills its waves
  }
  return best;
}

const char* lora_grad(const void* U, long long ldu, int R, const void* X, long long ldx, int C, int M, int n_splits,
                      float* partial, int* counters, float* out, long long ldo, cudaStream_t stream) {
  if (R <= 0 || R > 128 || (R % 8)) return "lora_grad: R must be a multiple of 8, at most 128";
  if ((C % 8) || (ldx % 8) || (ldu % 8) || (ldo % 4)) return "lora_grad: C, ldx, ldu must be multiples of 8 (ldo of 4)";
  if ((reinterpret_cast<uintptr_t>(U) & 15) || (reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return "lora_grad: operands must be 16-byte aligned";
  if (M <= 0 || C <= 0) return nullptr;
  const int rt = (R + 15) / 16;
  const int rows_per_split = ((M + n_splits - 1) / n_splits + LG_ROWS - 1) / LG_ROWS * LG_ROWS;
  dim3 grid((C + LG_COLS - 1) / LG_COLS, n_splits);
  constexpr int smem = LG_STAGES * 2 * LG_TILE_BYTES;
#define FERRL_LG(RTV)                                                                                                 \
  case RTV: {                                                                                                         \
    if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(lora_grad_kernel<RTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                    smem) == cudaSuccess))                                            \
      return "lora_grad: cannot reserve shared memory";                                                               \
    lora_grad_kernel<RTV><<<grid, 128, smem, stream>>>(static_cast<const __nv_bfloat16*>(U), ldu, R,                  \
                                                       static_cast<const __nv_bfloat16*>(X), ldx, C, M, rows_per_split, \
                                                       partial, counters, out, ldo);                                  \
    break;                                                                                                            \
  }
  switch (rt) {
    FERRL_LG(1) FERRL_LG(2) FERRL_LG(3) FERRL_LG(4) FERRL_LG(5) FERRL_LG(6) FERRL_LG(7) FERRL_LG(8)
    default: return "lora_grad: unsupported rank";
  }
#undef FERRL_LG
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "lora_grad launch failed";
}

}  // namespace ferrl
