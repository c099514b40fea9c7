// Chunked gated delta rule on tensor cores, forward and backward (GatedDeltaNet training and scoring).
//
// Reference: crates/ferrl/src/gdn.rs - gated_delta_rule_chunked (WY form, chunk 64) :451-556 and its
// block forward substitution ut_solve :400-431; the reference composes them from tensor ops with a
// Python-style loop over chunks and differentiates through that loop with the autograd tape.
//
// Per head, with chunk length C = 64, head dims 128 and for one chunk (rows = tokens of the chunk):
//   G   cumulative log decay inside the chunk, gamma = exp(G), D_ij = exp(G_i - G_j) (i >= j)
//   A   = tril(diag(beta) K K^T o D, -1),  T = (I + A)^-1
//   U   = T diag(beta) V,   W = T diag(gamma beta) K
//   Vn  = U - W S                              (S: state entering the chunk, [dk, dv] fp32)
//   O   = diag(gamma) Q S + tril(Q K^T o D) Vn
//   S'  = gamma_C S + (diag(gamma_C / gamma) K)^T Vn
// q and k arrive L2-normalised (q also scaled by 1/sqrt(dk)); those elementwise steps and their
// derivatives stay with the caller.
//
// Four kernels, all matrix products on the tensor cores (wmma m16n16k8, tf32 operands, fp32
// accumulation; operands are read as fp32 from shared or straight from global memory):
//   gdn_prep_kernel      one CTA per (chunk, head): G, T (forward substitution), U, W
//   gdn_scan_fwd_kernel  one CTA per head, chunks in order, state resident in shared memory: Vn, O, S'
//   gdn_scan_bwd_kernel  one CTA per head, chunks in reverse, dS resident: dVn and the dS recursion
//   gdn_chunk_bwd_kernel one CTA per (chunk, head): everything that does not cross chunks - dq, dk, dv,
//                        dbeta and dG (the caller turns dG into dg with a reverse cumulative sum)
// The two scans are the only sequential parts; the forward saves the entering state and Vn of every
// chunk when a backward will follow.
#include <cuda_runtime.h>
#include <mma.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"

namespace ferrl {

namespace {

namespace wm = nvcuda::wmma;
constexpr int GC = 64;      // chunk length
constexpr int GD = 128;     // key and value head dim

// Cm[M, N] (+)= op(A)[M, K] * op(B)[K, N] on the tensor cores; every pointer may be shared or global
// fp32, leading dimensions in floats (multiples of 4, 32-byte aligned tiles).  AT: A is stored [K, M];
// BT: B is stored [N, K].  Called by the whole CTA; the caller synchronises before it uses Cm.
template <bool AT, bool BT, bool ACC>
__device__ __forceinline__ void mm(float* Cm, int ldc, const float* A, long long lda, const float* Bm, long long ldb, int M, int N, int K) {
  const int warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int tn = N / 16, tiles = (M / 16) * tn;
  for (int t = warp; t < tiles; t += nw) {
    const int i = t / tn, j = t - i * tn;
    wm::fragment<wm::accumulator, 16, 16, 8, float> c;
    if (ACC) wm::load_matrix_sync(c, Cm + i * 16 * ldc + j * 16, ldc, wm::mem_row_major);
    else wm::fill_fragment(c, 0.f);
    for (int k = 0; k < K; k += 8) {
      if (!AT && !BT) {
        wm::fragment<wm::matrix_a, 16, 16, 8, wm::precision::tf32, wm::row_major> a;
        wm::fragment<wm::matrix_b, 16, 16, 8, wm::precision::tf32, wm::row_major> b;
        wm::load_matrix_sync(a, A + static_cast<long long>(i) * 16 * lda + k, static_cast<unsigned>(lda));
        wm::load_matrix_sync(b, Bm + static_cast<long long>(k) * ldb + j * 16, static_cast<unsigned>(ldb));
#pragma unroll
        for (int e = 0; e < a.num_elements; ++e) a.x[e] = wm::__float_to_tf32(a.x[e]);
#pragma unroll
        for (int e = 0; e < b.num_elements; ++e) b.x[e] = wm::__float_to_tf32(b.x[e]);
        wm::mma_sync(c, a, b, c);
      } else if (!AT && BT) {
        wm::fragment<wm::matrix_a, 16, 16, 8, wm::precision::tf32, wm::row_major> a;
        wm::fragment<wm::matrix_b, 16, 16, 8, wm::precision::tf32, wm::col_major> b;
        wm::load_matrix_sync(a, A + static_cast<long long>(i) * 16 * lda + k, static_cast<unsigned>(lda));
        wm::load_matrix_sync(b, Bm + static_cast<long long>(j) * 16 * ldb + k, static_cast<unsigned>(ldb));
#pragma unroll
        for (int e = 0; e < a.num_elements; ++e) a.x[e] = wm::__float_to_tf32(a.x[e]);
#pragma unroll
        for (int e = 0; e < b.num_elements; ++e) b.x[e] = wm::__float_to_tf32(b.x[e]);
        wm::mma_sync(c, a, b, c);
      } else if (AT && !BT) {
        wm::fragment<wm::matrix_a, 16, 16, 8, wm::precision::tf32, wm::col_major> a;
        wm::fragment<wm::matrix_b, 16, 16, 8, wm::precision::tf32, wm::row_major> b;
        wm::load_matrix_sync(a, A + static_cast<long long>(k) * lda + i * 16, static_cast<unsigned>(lda));
        wm::load_matrix_sync(b, Bm + static_cast<long long>(k) * ldb + j * 16, static_cast<unsigned>(ldb));
#pragma unroll
        for (int e = 0; e < a.num_elements; ++e) a.x[e] = wm::__float_to_tf32(a.x[e]);
#pragma unroll
        for (int e = 0; e < b.num_elements; ++e) b.x[e] = wm::__float_to_tf32(b.x[e]);
        wm::mma_sync(c, a, b, c);
      } else {
        wm::fragment<wm::matrix_a, 16, 16, 8, wm::precision::tf32, wm::col_major> a;
        wm::fragment<wm::matrix_b, 16, 16, 8, wm::precision::tf32, wm::col_major> b;
        wm::load_matrix_sync(a, A + static_cast<long long>(k) * lda + i * 16, static_cast<unsigned>(lda));
        wm::load_matrix_sync(b, Bm + static_cast<long long>(j) * 16 * ldb + k, static_cast<unsigned>(ldb));
#pragma unroll
        for (int e = 0; e < a.num_elements; ++e) a.x[e] = wm::__float_to_tf32(a.x[e]);
#pragma unroll
        for (int e = 0; e < b.num_elements; ++e) b.x[e] = wm::__float_to_tf32(b.x[e]);
        wm::mma_sync(c, a, b, c);
      }
    }
    wm::store_matrix_sync(Cm + i * 16 * ldc + j * 16, c, ldc, wm::mem_row_major);
  }
}

struct GdnDims {
  int B, T, Hk, Hv, n;        // T is a multiple of GC, n = T / GC chunks
};
// row pointer helpers: q,k are [B, T, Hk, GD], v/out/dO [B, T, Hv, GD], g/beta [B, T, Hv]
__device__ __forceinline__ long long qk_off(const GdnDims& d, int b, int t, int hk) {
  return ((static_cast<long long>(b) * d.T + t) * d.Hk + hk) * GD;
}
__device__ __forceinline__ long long v_off(const GdnDims& d, int b, int t, int hv) {
  return ((static_cast<long long>(b) * d.T + t) * d.Hv + hv) * GD;
}
__device__ __forceinline__ long long ch_off(const GdnDims& d, int b, int hv, int c) {      // chunk-indexed saves
  return (static_cast<long long>(b) * d.Hv + hv) * d.n + c;
}

// ---------------------------------------------------------------------------------------------
// prep: G, T, U, W of one chunk.  Shared: three [64, 64] matrices and two vectors.
__global__ void __launch_bounds__(256)
gdn_prep_kernel(const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ g,
                const float* __restrict__ beta, GdnDims d, float* __restrict__ Gc, float* __restrict__ Tm,
                float* __restrict__ U, float* __restrict__ W) {
  extern __shared__ __align__(128) float sm[];
  float* Y1 = sm;                  // K K^T, then A
  float* Y2 = Y1 + GC * GC;        // T
  float* Y3 = Y2 + GC * GC;        // T diag(beta), then T diag(gamma beta)
  float* Gs = Y3 + GC * GC;
  float* bs = Gs + GC;
  const int c = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / (d.Hv / d.Hk);
  const int tid = threadIdx.x;
  const long long ldk = static_cast<long long>(d.Hk) * GD, ldv = static_cast<long long>(d.Hv) * GD;
  const float* kg = k + qk_off(d, b, c * GC, hk);
  const float* vg = v + v_off(d, b, c * GC, hv);
  if (tid < GC) bs[tid] = beta[(static_cast<long long>(b) * d.T + c * GC + tid) * d.Hv + hv];
  if (tid == 0) {
    float acc = 0.f;
    for (int i = 0; i < GC; ++i) {
      acc += g[(static_cast<long long>(b) * d.T + c * GC + i) * d.Hv + hv];
      Gs[i] = acc;
    }
  }
  mm<false, true, false>(Y1, GC, kg, ldk, kg, ldk, GC, GC, GD);
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int i = e / GC, j = e - i * GC;
    Y1[e] = (i > j) ? bs[i] * Y1[e] * __expf(Gs[i] - Gs[j]) : 0.f;
    Y2[e] = (i == j) ? 1.f : 0.f;
  }
  __syncthreads();
  // T = (I + A)^-1 by forward substitution: row i of T is e_i - sum_{j<i} A[i][j] T[j][:]
  for (int i = 1; i < GC; ++i) {
    if (tid < GC) {
      float acc = (tid == i) ? 1.f : 0.f;
      for (int j = 0; j < i; ++j) acc -= Y1[i * GC + j] * Y2[j * GC + tid];
      Y2[i * GC + tid] = acc;
    }
    __syncthreads();
  }
  const long long co = ch_off(d, b, hv, c);
  for (int e = tid; e < GC * GC; e += 256) {
    const int j = e % GC;
    Tm[co * GC * GC + e] = Y2[e];
    Y3[e] = Y2[e] * bs[j];
  }
  if (tid < GC) Gc[co * GC + tid] = Gs[tid];
  __syncthreads();
  mm<false, false, false>(U + co * GC * GD, GD, Y3, GC, vg, ldv, GC, GD, GC);
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int j = e % GC;
    Y3[e] = Y2[e] * bs[j] * __expf(Gs[j]);
  }
  __syncthreads();
  mm<false, false, false>(W + co * GC * GD, GD, Y3, GC, kg, ldk, GC, GD, GC);
}

// ---------------------------------------------------------------------------------------------
// forward scan: one CTA per (head, batch), state in shared memory.
// Shared: S [128,128], Qs, Ks, Ws, Us [64,128] each, P [64,64], Gs [64].
__global__ void __launch_bounds__(256, 1)
gdn_scan_fwd_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ Gc,
                    const float* __restrict__ U, const float* __restrict__ W, const float* __restrict__ S0, GdnDims d,
                    float* __restrict__ out, float* __restrict__ S_out, float* __restrict__ Sin, float* __restrict__ Vn) {
  extern __shared__ __align__(128) float sm[];
  float* S = sm;
  float* Qs = S + GD * GD;
  float* Ks = Qs + GC * GD;
  float* Ws = Ks + GC * GD;
  float* Us = Ws + GC * GD;
  float* P = Us + GC * GD;
  float* Gs = P + GC * GC;
  const int hv = blockIdx.x, b = blockIdx.y;
  const int hk = hv / (d.Hv / d.Hk);
  const int tid = threadIdx.x;
  const long long bh = static_cast<long long>(b) * d.Hv + hv;
  for (int e = tid; e < GD * GD; e += 256) S[e] = S0 ? S0[bh * GD * GD + e] : 0.f;
  for (int c = 0; c < d.n; ++c) {
    const long long co = ch_off(d, b, hv, c);
    __syncthreads();
    for (int e = tid; e < GC * GD / 4; e += 256) {
      const int i = e / (GD / 4), x = e - i * (GD / 4);
      reinterpret_cast<float4*>(Qs)[e] = reinterpret_cast<const float4*>(q + qk_off(d, b, c * GC + i, hk))[x];
      reinterpret_cast<float4*>(Ks)[e] = reinterpret_cast<const float4*>(k + qk_off(d, b, c * GC + i, hk))[x];
      float4 w = reinterpret_cast<const float4*>(W + co * GC * GD)[e];
      reinterpret_cast<float4*>(Ws)[e] = make_float4(-w.x, -w.y, -w.z, -w.w);
      reinterpret_cast<float4*>(Us)[e] = reinterpret_cast<const float4*>(U + co * GC * GD)[e];
    }
    if (tid < GC) Gs[tid] = Gc[co * GC + tid];
    if (Sin)
      for (int e = tid; e < GD * GD / 4; e += 256)
        reinterpret_cast<float4*>(Sin + co * GD * GD)[e] = reinterpret_cast<const float4*>(S)[e];
    __syncthreads();
    mm<false, false, true>(Us, GD, Ws, GD, S, GD, GC, GD, GD);        // Vn = U - W S
    mm<false, true, false>(P, GC, Qs, GD, Ks, GD, GC, GC, GD);         // Q K^T
    __syncthreads();
    if (Vn)
      for (int e = tid; e < GC * GD / 4; e += 256)
        reinterpret_cast<float4*>(Vn + co * GC * GD)[e] = reinterpret_cast<const float4*>(Us)[e];
    for (int e = tid; e < GC * GC; e += 256) {
      const int i = e / GC, j = e - i * GC;
      P[e] = (i >= j) ? P[e] * __expf(Gs[i] - Gs[j]) : 0.f;
    }
    for (int e = tid; e < GC * GD; e += 256) Qs[e] *= __expf(Gs[e / GD]);
    __syncthreads();
    mm<false, false, false>(Ws, GD, Qs, GD, S, GD, GC, GD, GD);        // O = (gamma Q) S ...
    __syncthreads();
    mm<false, false, true>(Ws, GD, P, GC, Us, GD, GC, GD, GC);          // ... + P Vn
    __syncthreads();
    for (int e = tid; e < GC * GD / 4; e += 256) {
      const int i = e / (GD / 4), x = e - i * (GD / 4);
      reinterpret_cast<float4*>(out + v_off(d, b, c * GC + i, hv))[x] = reinterpret_cast<const float4*>(Ws)[e];
    }
    const float glast = Gs[GC - 1];
    const float eg = __expf(glast);
    for (int e = tid; e < GD * GD; e += 256) S[e] *= eg;
    for (int e = tid; e < GC * GD; e += 256) Ks[e] *= __expf(glast - Gs[e / GD]);
    __syncthreads();
    mm<true, false, true>(S, GD, Ks, GD, Us, GD, GD, GD, GC);           // S += (K decayed)^T Vn
  }
  __syncthreads();
  for (int e = tid; e < GD * GD; e += 256) S_out[bh * GD * GD + e] = S[e];
}

// ---------------------------------------------------------------------------------------------
// backward scan: chunks in reverse, dS in shared memory.
//   dVn = P^T dO + Kdec dS',   dS = gamma_C dS' + (gamma Q)^T dO - W^T dVn
// Writes dVn and the dS' of every chunk (gradient of the state leaving it) for the chunk kernel.
__global__ void __launch_bounds__(256, 1)
gdn_scan_bwd_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ Gc,
                    const float* __restrict__ W, const float* __restrict__ dO, const float* __restrict__ dS_final, GdnDims d,
                    float* __restrict__ dVn, float* __restrict__ dSout, float* __restrict__ dS0) {
  extern __shared__ __align__(128) float sm[];
  float* dS = sm;
  float* Qs = dS + GD * GD;
  float* Ks = Qs + GC * GD;
  float* Os = Ks + GC * GD;
  float* X = Os + GC * GD;
  float* P = X + GC * GD;
  float* Gs = P + GC * GC;
  const int hv = blockIdx.x, b = blockIdx.y;
  const int hk = hv / (d.Hv / d.Hk);
  const int tid = threadIdx.x;
  const long long bh = static_cast<long long>(b) * d.Hv + hv;
  for (int e = tid; e < GD * GD; e += 256) dS[e] = dS_final ? dS_final[bh * GD * GD + e] : 0.f;
  for (int c = d.n - 1; c >= 0; --c) {
    const long long co = ch_off(d, b, hv, c);
    __syncthreads();
    for (int e = tid; e < GC * GD / 4; e += 256) {
      const int i = e / (GD / 4), x = e - i * (GD / 4);
      reinterpret_cast<float4*>(Qs)[e] = reinterpret_cast<const float4*>(q + qk_off(d, b, c * GC + i, hk))[x];
      reinterpret_cast<float4*>(Ks)[e] = reinterpret_cast<const float4*>(k + qk_off(d, b, c * GC + i, hk))[x];
      reinterpret_cast<float4*>(Os)[e] = reinterpret_cast<const float4*>(dO + v_off(d, b, c * GC + i, hv))[x];
    }
    if (tid < GC) Gs[tid] = Gc[co * GC + tid];
    for (int e = tid; e < GD * GD / 4; e += 256)
      reinterpret_cast<float4*>(dSout + co * GD * GD)[e] = reinterpret_cast<const float4*>(dS)[e];
    __syncthreads();
    mm<false, true, false>(P, GC, Qs, GD, Ks, GD, GC, GC, GD);
    __syncthreads();
    const float glast = Gs[GC - 1];
    for (int e = tid; e < GC * GC; e += 256) {
      const int i = e / GC, j = e - i * GC;
      P[e] = (i >= j) ? P[e] * __expf(Gs[i] - Gs[j]) : 0.f;
    }
    for (int e = tid; e < GC * GD; e += 256) Ks[e] *= __expf(glast - Gs[e / GD]);
    __syncthreads();
    mm<true, false, false>(X, GD, P, GC, Os, GD, GC, GD, GC);          // P^T dO
    __syncthreads();
    mm<false, false, true>(X, GD, Ks, GD, dS, GD, GC, GD, GD);          // + Kdec dS'
    __syncthreads();
    for (int e = tid; e < GC * GD / 4; e += 256)
      reinterpret_cast<float4*>(dVn + co * GC * GD)[e] = reinterpret_cast<const float4*>(X)[e];
    const float eg = __expf(glast);
    for (int e = tid; e < GD * GD; e += 256) dS[e] *= eg;
    for (int e = tid; e < GC * GD; e += 256) Qs[e] *= __expf(Gs[e / GD]);
    for (int e = tid; e < GC * GD / 4; e += 256) {                      // Ks <- -W
      float4 w = reinterpret_cast<const float4*>(W + co * GC * GD)[e];
      reinterpret_cast<float4*>(Ks)[e] = make_float4(-w.x, -w.y, -w.z, -w.w);
    }
    __syncthreads();
    mm<true, false, true>(dS, GD, Qs, GD, Os, GD, GD, GD, GC);          // + (gamma Q)^T dO
    __syncthreads();
    mm<true, false, true>(dS, GD, Ks, GD, X, GD, GD, GD, GC);           // - W^T dVn
  }
  __syncthreads();
  if (dS0)
    for (int e = tid; e < GD * GD; e += 256) dS0[bh * GD * GD + e] = dS[e];
}

// ---------------------------------------------------------------------------------------------
// everything of the backward that stays inside a chunk.  Shared: E1, E2, E3 [64,128]; Y1, Y2, Y3
// [64,64]; vectors.  Operands that are plain inputs (q, k, v, dO, Vn, dVn, T, Sin, dSout) are read
// by the tensor-core loads straight from global memory.
__device__ __forceinline__ float block_sum256(float v, float* red) {
  return block_sum(v, red);
}

__global__ void __launch_bounds__(256, 1)
gdn_chunk_bwd_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                     const float* __restrict__ beta, const float* __restrict__ Gc, const float* __restrict__ Tm,
                     const float* __restrict__ Vn, const float* __restrict__ dVn, const float* __restrict__ Sin,
                     const float* __restrict__ dSout, const float* __restrict__ dO, GdnDims d, float* __restrict__ dq,
                     float* __restrict__ dk, float* __restrict__ dv, float* __restrict__ dbeta, float* __restrict__ dG) {
  extern __shared__ __align__(128) float sm[];
  float* E1 = sm;
  float* E2 = E1 + GC * GD;
  float* E3 = E2 + GC * GD;
  float* Y1 = E3 + GC * GD;
  float* Y2 = Y1 + GC * GC;
  float* Y3 = Y2 + GC * GC;
  float* Gs = Y3 + GC * GC;       // [64]
  float* bs = Gs + GC;            // [64]
  float* dGs = bs + GC;           // [64] accumulates dG
  float* dbs = dGs + GC;          // [64] accumulates dbeta
  float* red = dbs + GC;          // [32]
  const int c = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / (d.Hv / d.Hk);
  const int tid = threadIdx.x;
  const long long ldk = static_cast<long long>(d.Hk) * GD, ldv = static_cast<long long>(d.Hv) * GD;
  const long long co = ch_off(d, b, hv, c);
  const float* qg = q + qk_off(d, b, c * GC, hk);
  const float* kg = k + qk_off(d, b, c * GC, hk);
  const float* vg = v + v_off(d, b, c * GC, hv);
  const float* og = dO + v_off(d, b, c * GC, hv);
  const float* Tg = Tm + co * GC * GC;
  const float* Vng = Vn + co * GC * GD;
  const float* dVng = dVn + co * GC * GD;
  const float* Sg = Sin + co * GD * GD;
  const float* dSg = dSout + co * GD * GD;
  if (tid < GC) {
    Gs[tid] = Gc[co * GC + tid];
    bs[tid] = beta[(static_cast<long long>(b) * d.T + c * GC + tid) * d.Hv + hv];
    dGs[tid] = 0.f;
    dbs[tid] = 0.f;
  }
  __syncthreads();
  const float glast = Gs[GC - 1];

  // ---- 1. dQ = gamma o (dO Sin^T) + (dP o D) K;  dG from gamma in O and from D in P
  mm<false, true, false>(E1, GD, og, ldv, Sg, GD, GC, GD, GD);         // dO Sin^T            [64, dk]
  mm<false, true, false>(Y1, GC, og, ldv, Vng, GD, GC, GC, GD);        // dO Vn^T  = dP       [64, 64]
  mm<false, true, false>(Y2, GC, qg, ldk, kg, ldk, GC, GC, GD);        // Q K^T
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int i = e / GC, j = e - i * GC;
    const float dpd = (i >= j) ? Y1[e] * __expf(Gs[i] - Gs[j]) : 0.f;
    Y1[e] = dpd;                       // dP o D
    Y2[e] = dpd * Y2[e];               // M_P = dP o D o (Q K^T)
  }
  __syncthreads();
  if (tid < GC) {                      // row sums minus column sums of M_P, and the gamma-in-O term
    float rs = 0.f, cs = 0.f;
    for (int j = 0; j < GC; ++j) {
      rs += Y2[tid * GC + j];
      cs += Y2[j * GC + tid];
    }
    const float eg = __expf(Gs[tid]);
    float t = 0.f;
    for (int x = 0; x < GD; ++x) t += qg[tid * ldk + x] * E1[tid * GD + x];
    dGs[tid] += rs - cs + eg * t;
  }
  __syncthreads();
  for (int e = tid; e < GC * GD; e += 256) E1[e] *= __expf(Gs[e / GD]);
  __syncthreads();
  mm<false, false, true>(E1, GD, Y1, GC, kg, ldk, GC, GD, GC);
  __syncthreads();
  for (int e = tid; e < GC * GD / 4; e += 256) {
    const int i = e / (GD / 4), x = e - i * (GD / 4);
    reinterpret_cast<float4*>(dq + v_off(d, b, c * GC + i, hv))[x] = reinterpret_cast<const float4*>(E1)[e];
  }
  // ---- 2. dK (first part) = (dP o D)^T Q + (gamma_C / gamma) o (Vn dS'^T); dG from the decayed K in S'
  mm<false, true, false>(E2, GD, Vng, GD, dSg, GD, GC, GD, GD);        // Vn dS'^T             [64, dk]
  __syncthreads();
  if (tid < GC) {
    float t = 0.f;
    for (int x = 0; x < GD; ++x) t += kg[tid * ldk + x] * E2[tid * GD + x];
    const float r = __expf(glast - Gs[tid]) * t;
    dGs[tid] -= r;
    red[0] = 0.f;                      // (re)used below
    atomicAdd(&dGs[GC - 1], r);
  }
  __syncthreads();
  for (int e = tid; e < GC * GD; e += 256) E2[e] *= __expf(glast - Gs[e / GD]);
  __syncthreads();
  mm<true, false, true>(E2, GD, Y1, GC, qg, ldk, GC, GD, GC);
  // ---- gamma_C <Sin, dS'> goes to dG of the last row
  {
    float part = 0.f;
    for (int e = tid; e < GD * GD; e += 256) part += Sg[e] * dSg[e];
    const float tot = block_sum256(part, red);
    if (tid == 0) dGs[GC - 1] += __expf(glast) * tot;
  }
  __syncthreads();
  // ---- 3. dW = -dVn Sin^T
  mm<false, true, false>(E3, GD, dVng, GD, Sg, GD, GC, GD, GD);
  __syncthreads();
  for (int e = tid; e < GC * GD; e += 256) E3[e] = -E3[e];
  __syncthreads();
  // ---- 4. dT = (dVn V^T) diag(beta) + (dW K^T) diag(gamma beta)
  mm<false, true, false>(Y1, GC, dVng, GD, vg, ldv, GC, GC, GD);
  mm<false, true, false>(Y2, GC, E3, GD, kg, ldk, GC, GC, GD);
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int j = e % GC;
    Y1[e] = bs[j] * (Y1[e] + __expf(Gs[j]) * Y2[e]);
  }
  __syncthreads();
  // ---- 5. dVb = T^T dVn -> dV, dbeta
  mm<true, false, false>(E1, GD, Tg, GC, dVng, GD, GC, GD, GC);
  __syncthreads();
  if (tid < GC) {
    float t = 0.f;
    for (int x = 0; x < GD; ++x) t += E1[tid * GD + x] * vg[tid * ldv + x];
    dbs[tid] += t;
  }
  for (int e = tid; e < GC * GD / 4; e += 256) {
    const int i = e / (GD / 4), x = e - i * (GD / 4);
    float4 t = reinterpret_cast<const float4*>(E1)[e];
    const float bi = bs[i];
    reinterpret_cast<float4*>(dv + v_off(d, b, c * GC + i, hv))[x] = make_float4(t.x * bi, t.y * bi, t.z * bi, t.w * bi);
  }
  __syncthreads();
  // ---- 6. d(gamma Kb) = T^T dW
  mm<true, false, false>(E1, GD, Tg, GC, E3, GD, GC, GD, GC);
  // ---- 7. dA = -tril_strict(T^T dT T^T), taken with D; dG from D in A
  mm<true, false, false>(Y2, GC, Tg, GC, Y1, GC, GC, GC, GC);
  __syncthreads();
  mm<false, true, false>(Y3, GC, Y2, GC, Tg, GC, GC, GC, GC);
  mm<false, true, false>(Y2, GC, kg, ldk, kg, ldk, GC, GC, GD);        // K K^T
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int i = e / GC, j = e - i * GC;
    const float dad = (i > j) ? -Y3[e] * __expf(Gs[i] - Gs[j]) : 0.f;
    Y1[e] = dad;                       // dA o D
    Y2[e] = dad * bs[i] * Y2[e];       // M_A = dA o A
  }
  __syncthreads();
  if (tid < GC) {
    float rs = 0.f, cs = 0.f;
    for (int j = 0; j < GC; ++j) {
      rs += Y2[tid * GC + j];
      cs += Y2[j * GC + tid];
    }
    // gamma in W: sum_x d(gamma Kb)[i][x] * gamma_i beta_i K[i][x]
    float t = 0.f;
    for (int x = 0; x < GD; ++x) t += E1[tid * GD + x] * kg[tid * ldk + x];
    const float eg = __expf(Gs[tid]);
    dGs[tid] += rs - cs + eg * bs[tid] * t;
    // beta in M_A: A_ij = beta_i (K K^T o D)_ij  ->  dbeta_i += sum_j dA_ij A_ij / beta_i
    dbs[tid] += (bs[tid] != 0.f) ? rs / bs[tid] : 0.f;
  }
  __syncthreads();
  // ---- 8. dKb = (dA o D) K + gamma o d(gamma Kb)
  for (int e = tid; e < GC * GD; e += 256) E1[e] *= __expf(Gs[e / GD]);
  __syncthreads();
  mm<false, false, true>(E1, GD, Y1, GC, kg, ldk, GC, GD, GC);
  __syncthreads();
  if (tid < GC) {
    float t = 0.f;
    for (int x = 0; x < GD; ++x) t += E1[tid * GD + x] * kg[tid * ldk + x];
    dbs[tid] += t;
  }
  // ---- 9. dK (second part) = ((dA o D) with rows scaled by beta)^T K;  dK = E2 + beta o dKb
  for (int e = tid; e < GC * GC; e += 256) Y1[e] *= bs[e / GC];
  __syncthreads();
  mm<true, false, true>(E2, GD, Y1, GC, kg, ldk, GC, GD, GC);
  __syncthreads();
  for (int e = tid; e < GC * GD / 4; e += 256) {
    const int i = e / (GD / 4), x = e - i * (GD / 4);
    const float4 a = reinterpret_cast<const float4*>(E2)[e], t = reinterpret_cast<const float4*>(E1)[e];
    const float bi = bs[i];
    reinterpret_cast<float4*>(dk + v_off(d, b, c * GC + i, hv))[x] =
        make_float4(a.x + bi * t.x, a.y + bi * t.y, a.z + bi * t.z, a.w + bi * t.w);
  }
  if (tid < GC) {
    const long long o = (static_cast<long long>(b) * d.T + c * GC + tid) * d.Hv + hv;
    dG[o] = dGs[tid];
    dbeta[o] = dbs[tid];
  }
}

constexpr size_t kPrepSmem = (3 * GC * GC + 2 * GC) * sizeof(float);
constexpr size_t kScanSmem = (GD * GD + 4 * GC * GD + GC * GC + GC) * sizeof(float);
constexpr size_t kChunkBwdSmem = (3 * GC * GD + 3 * GC * GC + 4 * GC + 32) * sizeof(float);

}  // namespace

const char* gdn_tc_forward(const float* q, const float* k, const float* v, const float* g, const float* beta, const float* S0,
                           int B, int T, int Hk, int Hv, float* Gc, float* Tm, float* U, float* W, float* out,
                           float* S_out, float* Sin, float* Vn, cudaStream_t stream) {
  if (T % GC) return "gdn_tc: the sequence length must be a multiple of 64 (pad with beta = 0, g = 0)";
  if (Hk <= 0 || Hv % Hk) return "gdn_tc: value heads must be a multiple of key heads";
  if (B == 0 || T == 0) return nullptr;
  GdnDims d{B, T, Hk, Hv, T / GC};
  if (!FERRL_ONCE_PER_DEVICE(
          cudaFuncSetAttribute(gdn_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPrepSmem)) == cudaSuccess &&
          cudaFuncSetAttribute(gdn_scan_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kScanSmem)) == cudaSuccess))
    return "gdn_tc: cannot reserve shared memory";
  gdn_prep_kernel<<<dim3(d.n, Hv, B), 256, kPrepSmem, stream>>>(k, v, g, beta, d, Gc, Tm, U, W);
  count_launch();
  gdn_scan_fwd_kernel<<<dim3(Hv, B), 256, kScanSmem, stream>>>(q, k, Gc, U, W, S0, d, out, S_out, Sin, Vn);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_tc forward launch failed";
}

const char* gdn_tc_backward(const float* q, const float* k, const float* v, const float* beta, const float* Gc,
                            const float* Tm, const float* W, const float* Vn, const float* Sin, const float* dO,
                            const float* dS_final, int B, int T, int Hk, int Hv, float* dVn, float* dSout, float* dq,
                            float* dk, float* dv, float* dbeta, float* dG, float* dS0, cudaStream_t stream) {
  if (T % GC) return "gdn_tc: the sequence length must be a multiple of 64";
  if (Hk <= 0 || Hv % Hk) return "gdn_tc: value heads must be a multiple of key heads";
  if (B == 0 || T == 0) return nullptr;
  GdnDims d{B, T, Hk, Hv, T / GC};
  if (!FERRL_ONCE_PER_DEVICE(
          cudaFuncSetAttribute(gdn_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kScanSmem)) == cudaSuccess &&
          cudaFuncSetAttribute(gdn_chunk_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kChunkBwdSmem)) == cudaSuccess))
    return "gdn_tc: cannot reserve shared memory";
  gdn_scan_bwd_kernel<<<dim3(Hv, B), 256, kScanSmem, stream>>>(q, k, Gc, W, dO, dS_final, d, dVn, dSout, dS0);
  count_launch();
  gdn_chunk_bwd_kernel<<<dim3(d.n, Hv, B), 256, kChunkBwdSmem, stream>>>(q, k, v, beta, Gc, Tm, Vn, dVn, Sin, dSout, dO, d, dq,
                                                                         dk, dv, dbeta, dG);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_tc backward launch failed";
}

}  // namespace ferrl
