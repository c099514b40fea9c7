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
// All matrix products run on the tensor cores (wmma m16n16k8, tf32 operands, fp32 accumulation).  Only the
// two products per chunk that carry the state are sequential; everything else is one CTA per (chunk, head):
//   gdn_prep_kernel       G, T (forward substitution), U, Wn = -W, Kd = diag(gamma_C / gamma) K
//   gdn_scan_kernel<fwd>  one CTA per (head, slice of the value columns), chunks in order, state in shared
//                         memory: Vn = U + Wn S and S' = gamma_C S + Kd^T Vn; saves the entering state of each chunk
//   gdn_out_kernel        O of a chunk from its saved entering state
//   gdn_bwd_prep_kernel   X0 = P^T dO and Y0 = (gamma Q)^T dO
//   gdn_scan_kernel<bwd>  chunks in reverse: dVn = X0 + Kd dS', dS = gamma_C dS' + Y0 + Wn^T dVn
//   gdn_bwd_state_kernel  the chunk-local products with the saved states: dW, the state parts of dq, dk and dG
//   gdn_bwd_intra_kernel  everything else inside a chunk: dq, dk, dv, dbeta and dG (the caller turns dG into dg
//                         with a reverse cumulative sum inside each chunk)
#include <cuda_runtime.h>
#include <mma.h>
#include <stdint.h>

#include <type_traits>

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
#pragma unroll 4
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
// Shared-memory tiles carry a padded leading dimension so that the tensor-core fragment loads spread
// over the banks: an operand read "row by 4 columns" (A row-major, B column-major) wants ld = 4 mod 32,
// one read "4 rows by column" (B row-major, A column-major) wants ld = 8 mod 32.
constexpr int LD4 = GD + 4;     // 132
constexpr int LD8 = GD + 8;     // 136

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// rows x cols floats (cols a multiple of 4) from global (row stride lds) into shared (row stride ldd), whole CTA
__device__ __forceinline__ void tile_async(float* dst, int ldd, const float* src, long long lds, int rows, int cols) {
  const int c4 = cols >> 2;
  for (int e = threadIdx.x; e < rows * c4; e += blockDim.x) {
    const int r = e / c4, x = e - r * c4;
    cp_async16(dst + r * ldd + x * 4, src + r * lds + x * 4);
  }
}

// one 16x16 accumulator tile: c += op(A)[16, K] * op(B)[K, 16], k loop unrolled so the fragment loads overlap.
// A points at the tile's first row (AT: first column of the stored [K, M] matrix), B likewise.  The fp32 operands
// go to the tensor cores as they are: the tf32 path reads the top 19 bits (truncation instead of the
// round-to-nearest conversion, which would cost as many instructions as the loads themselves).
template <int K, bool AT, bool BT>
__device__ __forceinline__ void tile_mma(wm::fragment<wm::accumulator, 16, 16, 8, float>& c, const float* A, int lda,
                                         const float* Bm, int ldb) {
  using FA = typename std::conditional<AT, wm::fragment<wm::matrix_a, 16, 16, 8, wm::precision::tf32, wm::col_major>,
                                       wm::fragment<wm::matrix_a, 16, 16, 8, wm::precision::tf32, wm::row_major>>::type;
  using FB = typename std::conditional<BT, wm::fragment<wm::matrix_b, 16, 16, 8, wm::precision::tf32, wm::col_major>,
                                       wm::fragment<wm::matrix_b, 16, 16, 8, wm::precision::tf32, wm::row_major>>::type;
#pragma unroll
  for (int k = 0; k < K; k += 8) {
    FA a;
    FB b;
    wm::load_matrix_sync(a, AT ? A + k * lda : A + k, lda);
    wm::load_matrix_sync(b, BT ? Bm + k : Bm + k * ldb, ldb);
    wm::mma_sync(c, a, b, c);
  }
}

// ---------------------------------------------------------------------------------------------
// prep: per chunk G, T, U, Wn = -W, Kd = diag(exp(G_C - G)) K and gl = G_C.
// T = (I + A)^-1 with A strictly lower triangular: column c of T depends on A and on that column's own
// earlier rows only, so thread c solves its column in registers (fully unrolled, four partial sums per row
// to shorten the dependent chain) with no synchronisation at all.
// Shared: A / scaled T [64, 68], T [64, 68], K [64, 132], V [64, 136], two vectors.
constexpr size_t kPrepSmem = (2 * GC * (GC + 4) + GC * (GD + 4) + GC * (GD + 8) + 2 * GC) * sizeof(float);

__global__ void __launch_bounds__(256, 2)
gdn_prep_kernel(const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ g,
                const float* __restrict__ beta, GdnDims d, float* __restrict__ Gc, float* __restrict__ gl,
                float* __restrict__ Tm, float* __restrict__ U, float* __restrict__ Wn, float* __restrict__ Kd) {
  constexpr int LY = GC + 4;
  extern __shared__ __align__(128) float sm[];
  float* Y1 = sm;                  // K K^T, then A, then T diag(beta), then -T diag(gamma beta)
  float* Y2 = Y1 + GC * LY;        // T
  float* Ks = Y2 + GC * LY;        // [64, 132]
  float* Vs = Ks + GC * LD4;       // [64, 136]
  float* Gs = Vs + GC * LD8;
  float* bs = Gs + GC;
  const int c = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / (d.Hv / d.Hk);
  const int tid = threadIdx.x, warp = tid >> 5;
  const long long ldk = static_cast<long long>(d.Hk) * GD, ldv = static_cast<long long>(d.Hv) * GD;
  const long long co = ch_off(d, b, hv, c);
  tile_async(Ks, LD4, k + qk_off(d, b, c * GC, hk), ldk, GC, GD);
  tile_async(Vs, LD8, v + v_off(d, b, c * GC, hv), ldv, GC, GD);
  cp_async_commit();
  if (tid < GC) bs[tid] = beta[(static_cast<long long>(b) * d.T + c * GC + tid) * d.Hv + hv];
  if (tid < 32) {                  // inclusive scan of 64 log decays by one warp
    const long long o = (static_cast<long long>(b) * d.T + c * GC) * d.Hv + hv;
    float a0 = g[o + static_cast<long long>(2 * tid) * d.Hv], a1 = g[o + static_cast<long long>(2 * tid + 1) * d.Hv];
    float sum = a0 + a1;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, sum, off);
      if (tid >= off) sum += t;
    }
    Gs[2 * tid + 1] = sum;
    Gs[2 * tid] = sum - a1;
  }
  cp_async_wait_all();
  __syncthreads();
  for (int t = warp; t < 16; t += 8) {                 // K K^T
    const int ti = t >> 2, tj = t & 3;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GD, false, true>(acc, Ks + ti * 16 * LD4, LD4, Ks + tj * 16 * LD4, LD4);
    wm::store_matrix_sync(Y1 + ti * 16 * LY + tj * 16, acc, LY, wm::mem_row_major);
  }
  __syncthreads();
  const float glast = Gs[GC - 1];
  for (int e = tid; e < GC * GC; e += 256) {
    const int i = e / GC, j = e - i * GC;
    Y1[i * LY + j] = (i > j) ? bs[i] * Y1[i * LY + j] * __expf(Gs[i] - Gs[j]) : 0.f;
  }
  // Kd = diag(exp(G_C - G)) K
  for (int e = tid; e < GC * GD / 4; e += 256) {
    const int i = e / (GD / 4), x = e - i * (GD / 4);
    const float4 t = *reinterpret_cast<const float4*>(Ks + i * LD4 + x * 4);
    const float f = __expf(glast - Gs[i]);
    reinterpret_cast<float4*>(Kd + co * GC * GD)[e] = make_float4(t.x * f, t.y * f, t.z * f, t.w * f);
  }
  __syncthreads();
  if (tid < GC) {
    // column tid of T: t[i] = [i == tid] - sum_{j<i} A[i][j] t[j]; rows above the diagonal stay zero
    float t[GC];
#pragma unroll
    for (int i = 0; i < GC; ++i) {
      float a0 = (i == tid) ? 1.f : 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int j = 0; j + 3 < i; j += 4) {
        const float4 a = *reinterpret_cast<const float4*>(Y1 + i * LY + j);
        a0 -= a.x * t[j];
        a1 -= a.y * t[j + 1];
        a2 -= a.z * t[j + 2];
        a3 -= a.w * t[j + 3];
      }
#pragma unroll
      for (int j = i & ~3; j < i; ++j) a0 -= Y1[i * LY + j] * t[j];
      t[i] = (a0 + a1) + (a2 + a3);
      Y2[i * LY + tid] = t[i];
    }
  }
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int i = e / GC, j = e - i * GC;
    const float tv = Y2[i * LY + j];
    Tm[co * GC * GC + e] = tv;
    Y1[i * LY + j] = tv * bs[j];
  }
  if (tid < GC) Gc[co * GC + tid] = Gs[tid];
  if (tid == 0) gl[co] = glast;
  __syncthreads();
  for (int t = warp; t < 32; t += 8) {                 // U = T diag(beta) V
    const int ti = t >> 3, tj = t & 7;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GC, false, false>(acc, Y1 + ti * 16 * LY, LY, Vs + tj * 16, LD8);
    wm::store_matrix_sync(U + co * GC * GD + ti * 16 * GD + tj * 16, acc, GD, wm::mem_row_major);
  }
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int i = e / GC, j = e - i * GC;
    Y1[i * LY + j] = -Y2[i * LY + j] * bs[j] * __expf(Gs[j]);
  }
  __syncthreads();
  for (int t = warp; t < 32; t += 8) {                 // Wn = -T diag(gamma beta) K
    const int ti = t >> 3, tj = t & 7;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GC, false, false>(acc, Y1 + ti * 16 * LY, LY, Ks + tj * 16, LD4);
    wm::store_matrix_sync(Wn + co * GC * GD + ti * 16 * GD + tj * 16, acc, GD, wm::mem_row_major);
  }
}

// ---------------------------------------------------------------------------------------------
// The two scans.  The state's value columns never mix (Vn[:, j] and S'[:, j] depend on S[:, j] only), so a CTA
// owns DV of the 128 value columns of one head and walks the chunks with two products per chunk:
//   forward   Vn  = U  + Wn S              S' = gamma_C S   + Kd^T Vn
//   backward  dVn = X0 + Kd dS'            dS = gamma_C dS' + Y0 + Wn^T dVn      (chunks in reverse)
// Both have the form  V = V0 + A1 R;  R = g R + R0 + A2^T V  with per-chunk [64,128] matrices A1, A2, a
// [64, DV] start V0 and (backward only) a [128, DV] addend R0.  A1, A2 and V0 of the next chunk are fetched with
// cp.async while the current chunk computes; everything elementwise was folded into the per-chunk kernels.
template <int DV>
struct ScanSmem {
  static constexpr int LS = DV + 8;                                   // B row-major operands: 8 mod 32
  static constexpr int R = GD * LS, A1 = 2 * GC * LD4, A2 = 2 * GC * LD8, V = 2 * GC * LS;
  static constexpr size_t BYTES = static_cast<size_t>(R + A1 + A2 + V) * sizeof(float);
};

constexpr int kScanThreads = 512;

template <int DV, bool BWD>
__global__ void __launch_bounds__(kScanThreads, 1)
gdn_scan_kernel(const float* __restrict__ A1g,    // [.., n, 64, 128]: Wn (forward) / Kd (backward)
                const float* __restrict__ A2g,    // [.., n, 64, 128]: Kd (forward) / Wn (backward)
                const float* __restrict__ V0g,    // [.., n, 64, 128]: U (forward) / X0 (backward)
                const float* __restrict__ R0g,    // backward: Y0 [.., n, 128, 128]; forward: null
                const float* __restrict__ gl,     // [.., n] last cumulative log decay of every chunk
                const float* __restrict__ Rinit,  // [.., 128, 128] initial state (S0 / dS_final) or null
                int n, int n_slices,
                float* __restrict__ Vout,         // [.., n, 64, 128]: Vn / dVn
                float* __restrict__ Rchunks,      // [.., n, 128, 128]: forward Sin[c] = state entering chunk c;
                                                  //                    backward dSout[c] = gradient of the state leaving c
                float* __restrict__ Rfinal) {     // [.., 128, 128]: S after the last chunk / dS0 (may be null)
  using SM = ScanSmem<DV>;
  constexpr int LS = SM::LS;
  extern __shared__ __align__(128) float sm[];
  float* Rs = sm;
  float* A1s = Rs + SM::R;
  float* A2s = A1s + SM::A1;
  float* Vs = A2s + SM::A2;
  __shared__ float gls[1024];
  const int slice = blockIdx.x % n_slices;
  const long long bh = blockIdx.x / n_slices + static_cast<long long>(blockIdx.y) * (gridDim.x / n_slices);
  const int col0 = slice * DV;
  const int tid = threadIdx.x, warp = tid >> 5;
  const long long cbase = bh * n;
  for (int e = tid; e < n; e += kScanThreads) gls[e] = gl[cbase + e];
  for (int e = tid; e < GD * DV; e += kScanThreads) {
    const int r = e / DV, x = e - r * DV;
    Rs[r * LS + x] = Rinit ? Rinit[bh * GD * GD + r * GD + col0 + x] : 0.f;
  }
  auto fetch = [&](int c, int buf) {
    const long long co = cbase + c;
    tile_async(A1s + buf * GC * LD4, LD4, A1g + co * GC * GD, GD, GC, GD);
    tile_async(A2s + buf * GC * LD8, LD8, A2g + co * GC * GD, GD, GC, GD);
    tile_async(Vs + buf * GC * LS, LS, V0g + co * GC * GD + col0, GD, GC, DV);
    cp_async_commit();
  };
  const int first = BWD ? n - 1 : 0, step = BWD ? -1 : 1;
  fetch(first, 0);
  __syncthreads();
  {  // the state as the first chunk sees it
    float* dst = Rchunks + (cbase + first) * GD * GD;
    for (int e = tid; e < GD * DV; e += kScanThreads) {
      const int r = e / DV, x = e - r * DV;
      dst[r * GD + col0 + x] = Rs[r * LS + x];
    }
  }
  constexpr int TN = DV / 16;
  for (int i = 0; i < n; ++i) {
    const int c = first + i * step, buf = i & 1;
    cp_async_wait_all();
    __syncthreads();                        // this chunk's tiles have landed; the other buffer and Rs are free
    if (i + 1 < n) fetch(c + step, buf ^ 1);
    const float* a1 = A1s + buf * GC * LD4;
    const float* a2 = A2s + buf * GC * LD8;
    float* vs = Vs + buf * GC * LS;
    const long long co = cbase + c;
    // V = V0 + A1 R    [64, DV], K = 128
    for (int t = warp; t < (GC / 16) * TN; t += kScanThreads / 32) {
      const int ti = t / TN, tj = t - ti * TN;
      wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
      wm::load_matrix_sync(acc, vs + ti * 16 * LS + tj * 16, LS, wm::mem_row_major);
      tile_mma<GD, false, false>(acc, a1 + ti * 16 * LD4, LD4, Rs + tj * 16, LS);
      wm::store_matrix_sync(vs + ti * 16 * LS + tj * 16, acc, LS, wm::mem_row_major);
      wm::store_matrix_sync(Vout + co * GC * GD + ti * 16 * GD + col0 + tj * 16, acc, GD, wm::mem_row_major);
    }
    __syncthreads();
    // R = g R (+ R0) + A2^T V    [128, DV], K = 64
    const float eg = __expf(gls[c]);
    const bool last = i + 1 == n;
    float* rdst = last ? (Rfinal ? Rfinal + bh * GD * GD : nullptr) : Rchunks + (cbase + c + step) * GD * GD;
    for (int t = warp; t < (GD / 16) * TN; t += kScanThreads / 32) {
      const int ti = t / TN, tj = t - ti * TN;
      wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
      wm::load_matrix_sync(acc, Rs + ti * 16 * LS + tj * 16, LS, wm::mem_row_major);
      if (BWD) {
        wm::fragment<wm::accumulator, 16, 16, 8, float> add;
        wm::load_matrix_sync(add, R0g + co * GD * GD + ti * 16 * GD + col0 + tj * 16, GD, wm::mem_row_major);
#pragma unroll
        for (int e = 0; e < acc.num_elements; ++e) acc.x[e] = acc.x[e] * eg + add.x[e];
      } else {
#pragma unroll
        for (int e = 0; e < acc.num_elements; ++e) acc.x[e] *= eg;
      }
      tile_mma<GC, true, false>(acc, a2 + ti * 16, LD8, vs + tj * 16, LS);
      wm::store_matrix_sync(Rs + ti * 16 * LS + tj * 16, acc, LS, wm::mem_row_major);
      if (rdst) wm::store_matrix_sync(rdst + ti * 16 * GD + col0 + tj * 16, acc, GD, wm::mem_row_major);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// output of one chunk from the saved entering state:  O = diag(gamma) Q Sin + tril(Q K^T o D) Vn
// Shared: Q, K [64, 132]; Sin [128, 136]; Vn [64, 136]; P [64, 68]; G [64].
constexpr int LP = GC + 4;      // 68
constexpr size_t kOutSmem = (2 * GC * LD4 + GD * LD8 + GC * LD8 + GC * LP + GC) * sizeof(float);

__global__ void __launch_bounds__(512, 1)
gdn_out_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ Gc,
               const float* __restrict__ Sin, const float* __restrict__ Vn, GdnDims d, float* __restrict__ out) {
  extern __shared__ __align__(128) float sm[];
  float* Qs = sm;
  float* Ks = Qs + GC * LD4;
  float* Ss = Ks + GC * LD4;
  float* Vs = Ss + GD * LD8;
  float* P = Vs + GC * LD8;
  float* Gs = P + GC * LP;
  const int c = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / (d.Hv / d.Hk);
  const int tid = threadIdx.x, warp = tid >> 5;
  const long long ldk = static_cast<long long>(d.Hk) * GD, ldv = static_cast<long long>(d.Hv) * GD;
  const long long co = ch_off(d, b, hv, c);
  tile_async(Qs, LD4, q + qk_off(d, b, c * GC, hk), ldk, GC, GD);
  tile_async(Ks, LD4, k + qk_off(d, b, c * GC, hk), ldk, GC, GD);
  cp_async_commit();
  tile_async(Ss, LD8, Sin + co * GD * GD, GD, GD, GD);
  tile_async(Vs, LD8, Vn + co * GC * GD, GD, GC, GD);
  cp_async_commit();
  if (tid < GC) Gs[tid] = Gc[co * GC + tid];
  asm volatile("cp.async.wait_group 1;" ::: "memory");
  __syncthreads();
  for (int t = warp; t < 16; t += 16) {                 // P = Q K^T
    const int ti = t >> 2, tj = t & 3;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GD, false, true>(acc, Qs + ti * 16 * LD4, LD4, Ks + tj * 16 * LD4, LD4);
    wm::store_matrix_sync(P + ti * 16 * LP + tj * 16, acc, LP, wm::mem_row_major);
  }
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 512) {
    const int i = e / GC, j = e - i * GC;
    P[i * LP + j] = (i >= j) ? P[i * LP + j] * __expf(Gs[i] - Gs[j]) : 0.f;
  }
  for (int e = tid; e < GC * GD; e += 512) {
    const int i = e / GD, x = e - i * GD;
    Qs[i * LD4 + x] *= __expf(Gs[i]);
  }
  cp_async_wait_all();
  __syncthreads();
  float* og = out + v_off(d, b, c * GC, hv);
  for (int t = warp; t < 32; t += 16) {                 // O = (gamma Q) Sin + P Vn
    const int ti = t >> 3, tj = t & 7;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GD, false, false>(acc, Qs + ti * 16 * LD4, LD4, Ss + tj * 16, LD8);
    tile_mma<GC, false, false>(acc, P + ti * 16 * LP, LP, Vs + tj * 16, LD8);
    wm::store_matrix_sync(og + static_cast<long long>(ti) * 16 * ldv + tj * 16, acc, static_cast<unsigned>(ldv), wm::mem_row_major);
  }
}

// ---------------------------------------------------------------------------------------------
// backward, chunk-local inputs of the reverse scan:  X0 = P^T dO  [64,128],  Y0 = (gamma Q)^T dO  [128,128]
// Shared: Q, K [64, 132]; dO [64, 136]; P [64, 72]; G [64].
constexpr int LP8 = GC + 8;     // 72
constexpr size_t kBwdPrepSmem = (2 * GC * LD4 + GC * LD8 + GC * LP8 + GC) * sizeof(float);

__global__ void __launch_bounds__(512, 1)
gdn_bwd_prep_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ Gc,
                    const float* __restrict__ dO, GdnDims d, float* __restrict__ X0, float* __restrict__ Y0) {
  extern __shared__ __align__(128) float sm[];
  float* Qs = sm;
  float* Ks = Qs + GC * LD4;
  float* Os = Ks + GC * LD4;
  float* P = Os + GC * LD8;
  float* Gs = P + GC * LP8;
  const int c = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / (d.Hv / d.Hk);
  const int tid = threadIdx.x, warp = tid >> 5;
  const long long ldk = static_cast<long long>(d.Hk) * GD, ldv = static_cast<long long>(d.Hv) * GD;
  const long long co = ch_off(d, b, hv, c);
  tile_async(Qs, LD4, q + qk_off(d, b, c * GC, hk), ldk, GC, GD);
  tile_async(Ks, LD4, k + qk_off(d, b, c * GC, hk), ldk, GC, GD);
  tile_async(Os, LD8, dO + v_off(d, b, c * GC, hv), ldv, GC, GD);
  cp_async_commit();
  if (tid < GC) Gs[tid] = Gc[co * GC + tid];
  cp_async_wait_all();
  __syncthreads();
  for (int t = warp; t < 16; t += 16) {
    const int ti = t >> 2, tj = t & 3;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GD, false, true>(acc, Qs + ti * 16 * LD4, LD4, Ks + tj * 16 * LD4, LD4);
    wm::store_matrix_sync(P + ti * 16 * LP8 + tj * 16, acc, LP8, wm::mem_row_major);
  }
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 512) {
    const int i = e / GC, j = e - i * GC;
    P[i * LP8 + j] = (i >= j) ? P[i * LP8 + j] * __expf(Gs[i] - Gs[j]) : 0.f;
  }
  for (int e = tid; e < GC * GD; e += 512) {
    const int i = e / GD, x = e - i * GD;
    Qs[i * LD4 + x] *= __expf(Gs[i]);
  }
  __syncthreads();
  for (int t = warp; t < 32; t += 16) {                 // X0 = P^T dO
    const int ti = t >> 3, tj = t & 7;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GC, true, false>(acc, P + ti * 16, LP8, Os + tj * 16, LD8);
    wm::store_matrix_sync(X0 + co * GC * GD + ti * 16 * GD + tj * 16, acc, GD, wm::mem_row_major);
  }
  for (int t = warp; t < 64; t += 16) {                 // Y0 = (gamma Q)^T dO
    const int ti = t >> 3, tj = t & 7;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GC, true, false>(acc, Qs + ti * 16, LD4, Os + tj * 16, LD8);
    wm::store_matrix_sync(Y0 + co * GD * GD + ti * 16 * GD + tj * 16, acc, GD, wm::mem_row_major);
  }
}

// ---------------------------------------------------------------------------------------------
// Backward, the part of a chunk that touches the states.  One CTA per (chunk, half of the key dims):
//   E1 = dO Sin^T    -> dq  = gamma o E1          (the chunk kernel adds (dP o D) K),  dG += gamma <Q, E1>
//   dW = -dVn Sin^T  -> global
//   E2 = Vn dS'^T    -> dk  = (gamma_C / gamma) o E2 (the chunk kernel adds the rest), R = <K, that>:
//                       dG -= R, dG[last] += sum R;   dG[last] += gamma_C <Sin, dS'>
// Shared: one half state [64 key dims, 132], one [64, 132] operand tile, one [64, 68] result, vectors.
constexpr size_t kBwdStateSmem = (2 * GC * LD4 + GC * LP + 3 * GC + 32) * sizeof(float);

__global__ void __launch_bounds__(256, 2)
gdn_bwd_state_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ Gc,
                     const float* __restrict__ Vn, const float* __restrict__ dVn, const float* __restrict__ Sin,
                     const float* __restrict__ dSout, const float* __restrict__ dO, GdnDims d, float* __restrict__ dq,
                     float* __restrict__ dk, float* __restrict__ dW, float* __restrict__ dGpart) {
  extern __shared__ __align__(128) float sm[];
  float* Sh = sm;                    // [64, LD4] rows = key dims of this half, cols = value dims
  float* X = Sh + GC * LD4;          // [64, LD4] dO, then dVn, then Vn
  float* E = X + GC * LD4;           // [64, LP]
  float* Gs = E + GC * LP;
  float* dGs = Gs + GC;
  float* Rv = dGs + GC;
  float* red = Rv + GC;
  const int c = blockIdx.x >> 1, half = blockIdx.x & 1, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / (d.Hv / d.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long ldk = static_cast<long long>(d.Hk) * GD, ldv = static_cast<long long>(d.Hv) * GD;
  const long long co = ch_off(d, b, hv, c);
  const int kc0 = half * GC;                                          // first key dim of this half
  const float* qg = q + qk_off(d, b, c * GC, hk) + kc0;
  const float* kg = k + qk_off(d, b, c * GC, hk) + kc0;
  const float* Sg = Sin + co * GD * GD + static_cast<long long>(kc0) * GD;
  const float* dSg = dSout + co * GD * GD + static_cast<long long>(kc0) * GD;
  tile_async(Sh, LD4, Sg, GD, GC, GD);
  tile_async(X, LD4, dO + v_off(d, b, c * GC, hv), ldv, GC, GD);
  cp_async_commit();
  if (tid < GC) {
    Gs[tid] = Gc[co * GC + tid];
    dGs[tid] = 0.f;
  }
  cp_async_wait_all();
  __syncthreads();
  const float glast = Gs[GC - 1];
  auto product = [&](bool negate_to_dW) {                              // [64, 64] = X Sh^T, K = 128
    for (int t = warp; t < 16; t += 8) {
      const int ti = t >> 2, tj = t & 3;
      wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
      wm::fill_fragment(acc, 0.f);
      tile_mma<GD, false, true>(acc, X + ti * 16 * LD4, LD4, Sh + tj * 16 * LD4, LD4);
      if (negate_to_dW) {
#pragma unroll
        for (int e = 0; e < acc.num_elements; ++e) acc.x[e] = -acc.x[e];
        wm::store_matrix_sync(dW + co * GC * GD + ti * 16 * GD + kc0 + tj * 16, acc, GD, wm::mem_row_major);
      } else {
        wm::store_matrix_sync(E + ti * 16 * LP + tj * 16, acc, LP, wm::mem_row_major);
      }
    }
  };
  // row i of E scaled by f(i) goes to dst[i][kc0 + x]; returns through dots[i] the scaled row's dot with src[i]
  auto scale_rows = [&](float* dst, const float* src, bool by_gamma, float* dots) {
    for (int i = warp * 8; i < warp * 8 + 8; ++i) {
      const float f = by_gamma ? __expf(Gs[i]) : __expf(glast - Gs[i]);
      const float e0 = f * E[i * LP + lane], e1 = f * E[i * LP + lane + 32];
      float* drow = dst + v_off(d, b, c * GC + i, hv) + kc0;
      drow[lane] = e0;
      drow[lane + 32] = e1;
      float dot = e0 * src[i * ldk + lane] + e1 * src[i * ldk + lane + 32];
      dot = warp_sum(dot);
      if (lane == 0) dots[i] = dot;
    }
  };
  product(false);                                                      // E1 = dO Sin^T
  __syncthreads();
  scale_rows(dq, qg, true, Rv);
  __syncthreads();
  if (tid < GC) dGs[tid] += Rv[tid];
  tile_async(X, LD4, dVn + co * GC * GD, GD, GC, GD);
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();
  product(true);                                                       // dW = -dVn Sin^T
  {                                                                    // gamma_C <Sin, dS'> over this half
    float part = 0.f;
    for (int e = tid; e < GC * GD / 4; e += 256) {
      const int r = e / (GD / 4), x = e - r * (GD / 4);
      const float4 a = *reinterpret_cast<const float4*>(Sh + r * LD4 + x * 4);
      const float4 g4 = reinterpret_cast<const float4*>(dSg + static_cast<long long>(r) * GD)[x];
      part += a.x * g4.x + a.y * g4.y + a.z * g4.z + a.w * g4.w;
    }
    const float tot = block_sum(part, red);
    if (tid == 0) dGs[GC - 1] += __expf(glast) * tot;
  }
  __syncthreads();
  tile_async(Sh, LD4, dSg, GD, GC, GD);
  tile_async(X, LD4, Vn + co * GC * GD, GD, GC, GD);
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();
  product(false);                                                      // E2 = Vn dS'^T
  __syncthreads();
  scale_rows(dk, kg, false, Rv);
  __syncthreads();
  if (tid < GC) dGs[tid] -= Rv[tid];
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int i = 0; i < GC; ++i) t += Rv[i];
    dGs[GC - 1] += t;
  }
  __syncthreads();
  if (tid < GC)
    dGpart[(static_cast<long long>(half) * d.B * d.T + static_cast<long long>(b) * d.T + c * GC + tid) * d.Hv + hv] = dGs[tid];
}

// ---------------------------------------------------------------------------------------------
// Backward, everything inside a chunk that does not touch the states.  With Z1 = dVn V^T, Z2 = dW K^T:
//   dP o D = tril(dO Vn^T) o D;   dq += (dP o D) K;   dk += (dP o D)^T Q
//   dT = (Z1 + Z2 diag(gamma)) diag(beta);   dA o D = -tril(T^T dT T^T, -1) o D;   Ab = diag(beta) (dA o D)
//   dv = (T diag(beta))^T dVn;   dk += Ab K + Ab^T K + (T diag(gamma beta))^T dW
//   dbeta_i = sum_k T_ki (Z1_ki + gamma_i Z2_ki) + sum_j (dA o D)_ij (K K^T)_ij
//   dG_i  += rowsum - colsum of (dP o D) o (Q K^T) and of Ab o (K K^T), + gamma_i beta_i sum_k T_ki Z2_ki
// The products Tᵀ dVn and Tᵀ dW never exist as tiles: their row dots are column sums over T o Z, and their
// contributions to dv and dk are products with pre-scaled copies of T.
// Shared: five [64, 132] tiles (Q, K, dO, Vn, dk accumulator; later V, K, dVn, dW), three [64, 68], vectors.
constexpr size_t kBwdIntraSmem = (5 * GC * LD4 + 3 * GC * LP + 6 * GC) * sizeof(float);
constexpr int kIntraThreads = 512;

__global__ void __launch_bounds__(kIntraThreads, 1)
gdn_bwd_intra_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                     const float* __restrict__ beta, const float* __restrict__ Gc, const float* __restrict__ Tm,
                     const float* __restrict__ Vn, const float* __restrict__ dVn, const float* __restrict__ dW,
                     const float* __restrict__ dO, const float* __restrict__ dGpart, GdnDims d, float* __restrict__ dq,
                     float* __restrict__ dk, float* __restrict__ dv, float* __restrict__ dbeta, float* __restrict__ dG) {
  extern __shared__ __align__(128) float sm[];
  float* tQ = sm;                     // Q, later V
  float* tK = tQ + GC * LD4;          // K
  float* tO = tK + GC * LD4;          // dO, later dVn
  float* tV = tO + GC * LD4;          // Vn, later dW
  float* tD = tV + GC * LD4;          // dk accumulator
  float* Y1 = tD + GC * LD4;
  float* Y2 = Y1 + GC * LP;
  float* Y3 = Y2 + GC * LP;
  float* Gs = Y3 + GC * LP;
  float* bs = Gs + GC;
  float* dGs = bs + GC;
  float* dbs = dGs + GC;
  float* s1 = dbs + GC;
  float* s2 = s1 + GC;
  constexpr int NW = kIntraThreads / 32;
  const int c = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / (d.Hv / d.Hk);
  const int tid = threadIdx.x, warp = tid >> 5;
  const long long ldk = static_cast<long long>(d.Hk) * GD, ldv = static_cast<long long>(d.Hv) * GD;
  const long long co = ch_off(d, b, hv, c);
  const long long vo = v_off(d, b, c * GC, hv);
  tile_async(tQ, LD4, q + qk_off(d, b, c * GC, hk), ldk, GC, GD);
  tile_async(tK, LD4, k + qk_off(d, b, c * GC, hk), ldk, GC, GD);
  tile_async(tO, LD4, dO + vo, ldv, GC, GD);
  tile_async(tV, LD4, Vn + co * GC * GD, GD, GC, GD);
  cp_async_commit();
  if (tid < GC) {
    const long long o = (static_cast<long long>(b) * d.T + c * GC + tid) * d.Hv + hv;
    Gs[tid] = Gc[co * GC + tid];
    bs[tid] = beta[o];
    dGs[tid] = dGpart[o] + dGpart[static_cast<long long>(d.B) * d.T * d.Hv + o];
    dbs[tid] = 0.f;
  }
  cp_async_wait_all();
  __syncthreads();
  // [64, 64] = A B^T with A, B [64, 128] tiles
  auto abt = [&](float* Y, const float* A, const float* Bt, int t0) {
    for (int t = warp - t0; t < 16 && t >= 0; t += NW) {
      const int ti = t >> 2, tj = t & 3;
      wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
      wm::fill_fragment(acc, 0.f);
      tile_mma<GD, false, true>(acc, A + ti * 16 * LD4, LD4, Bt + tj * 16 * LD4, LD4);
      wm::store_matrix_sync(Y + ti * 16 * LP + tj * 16, acc, LP, wm::mem_row_major);
    }
  };
  // ---- dP o D and its dG term
  abt(Y1, tO, tV, 0);                                                  // dO Vn^T   (warps 0..15 take one tile each)
  __syncthreads();
  abt(Y2, tQ, tK, 0);                                                  // Q K^T
  __syncthreads();
  for (int e = tid; e < GC * GC; e += kIntraThreads) {
    const int i = e / GC, j = e - i * GC;
    const float dpd = (i >= j) ? Y1[i * LP + j] * __expf(Gs[i] - Gs[j]) : 0.f;
    Y1[i * LP + j] = dpd;
    Y2[i * LP + j] *= dpd;
  }
  __syncthreads();
  if (tid < GC) {
    float rs = 0.f, cs = 0.f;
    for (int j = 0; j < GC; ++j) {
      rs += Y2[tid * LP + j];
      cs += Y2[j * LP + tid];
    }
    dGs[tid] += rs - cs;
  }
  // ---- dq = dq(state part) + (dP o D) K;  dk accumulator = dk(state part) + (dP o D)^T Q
  for (int t = warp; t < 64; t += NW) {
    const int which = t >> 5, tt = t & 31, ti = tt >> 3, tj = tt & 7;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    float* gsrc = (which ? dk : dq) + vo + static_cast<long long>(ti) * 16 * ldv + tj * 16;
    wm::load_matrix_sync(acc, gsrc, static_cast<unsigned>(ldv), wm::mem_row_major);
    if (which == 0) {
      tile_mma<GC, false, false>(acc, Y1 + ti * 16 * LP, LP, tK + tj * 16, LD4);
      wm::store_matrix_sync(gsrc, acc, static_cast<unsigned>(ldv), wm::mem_row_major);
    } else {
      tile_mma<GC, true, false>(acc, Y1 + ti * 16, LP, tQ + tj * 16, LD4);
      wm::store_matrix_sync(tD + ti * 16 * LD4 + tj * 16, acc, LD4, wm::mem_row_major);
    }
  }
  __syncthreads();
  // ---- second set of operands: V, dVn, dW, T
  tile_async(tQ, LD4, v + vo, ldv, GC, GD);
  tile_async(tO, LD4, dVn + co * GC * GD, GD, GC, GD);
  tile_async(tV, LD4, dW + co * GC * GD, GD, GC, GD);
  tile_async(Y3, LP, Tm + co * GC * GC, GC, GC, GC);
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();
  abt(Y2, tO, tQ, 0);                                                  // Z1 = dVn V^T
  __syncthreads();
  abt(Y1, tV, tK, 0);                                                  // Z2 = dW K^T
  __syncthreads();
  if (tid < GC) {                                                      // column sums of T o Z1, T o Z2
    float a1 = 0.f, a2 = 0.f;
    for (int kk = 0; kk < GC; ++kk) {
      const float t = Y3[kk * LP + tid];
      a1 += t * Y2[kk * LP + tid];
      a2 += t * Y1[kk * LP + tid];
    }
    const float eg = __expf(Gs[tid]);
    dbs[tid] += a1 + eg * a2;
    dGs[tid] += eg * bs[tid] * a2;
  }
  __syncthreads();
  for (int e = tid; e < GC * GC; e += kIntraThreads) {                 // dT
    const int i = e / GC, j = e - i * GC;
    Y1[i * LP + j] = bs[j] * (Y2[i * LP + j] + __expf(Gs[j]) * Y1[i * LP + j]);
  }
  __syncthreads();
  // ---- dA = -tril(T^T dT T^T, -1)
  for (int t = warp; t < 16; t += NW) {                                // Y2 = T^T dT
    const int ti = t >> 2, tj = t & 3;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GC, true, false>(acc, Y3 + ti * 16, LP, Y1 + tj * 16, LP);
    wm::store_matrix_sync(Y2 + ti * 16 * LP + tj * 16, acc, LP, wm::mem_row_major);
  }
  __syncthreads();
  for (int t = warp; t < 16; t += NW) {                                // Y1 = Y2 T^T
    const int ti = t >> 2, tj = t & 3;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GC, false, true>(acc, Y2 + ti * 16 * LP, LP, Y3 + tj * 16 * LP, LP);
    wm::store_matrix_sync(Y1 + ti * 16 * LP + tj * 16, acc, LP, wm::mem_row_major);
  }
  __syncthreads();
  abt(Y2, tK, tK, 0);                                                  // K K^T
  __syncthreads();
  for (int e = tid; e < GC * GC; e += kIntraThreads) {
    const int i = e / GC, j = e - i * GC;
    const float dad = (i > j) ? -Y1[i * LP + j] * __expf(Gs[i] - Gs[j]) : 0.f;
    Y2[i * LP + j] *= dad;                                             // (dA o D) o (K K^T)
    Y1[i * LP + j] = dad * bs[i];                                      // Ab = diag(beta) (dA o D)
  }
  __syncthreads();
  if (tid < GC) {
    float rs = 0.f, cs = 0.f;
    for (int j = 0; j < GC; ++j) {
      rs += Y2[tid * LP + j];
      cs += bs[j] * Y2[j * LP + tid];
    }
    dbs[tid] += rs;
    dGs[tid] += bs[tid] * rs - cs;
  }
  for (int e = tid; e < GC * GC; e += kIntraThreads) Y3[(e / GC) * LP + (e % GC)] *= bs[e % GC];     // T diag(beta)
  __syncthreads();
  for (int t = warp; t < 32; t += NW) {                                // dv = (T diag(beta))^T dVn
    const int ti = t >> 3, tj = t & 7;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GC, true, false>(acc, Y3 + ti * 16, LP, tO + tj * 16, LD4);
    wm::store_matrix_sync(dv + vo + static_cast<long long>(ti) * 16 * ldv + tj * 16, acc, static_cast<unsigned>(ldv), wm::mem_row_major);
  }
  __syncthreads();
  for (int e = tid; e < GC * GC; e += kIntraThreads) Y3[(e / GC) * LP + (e % GC)] *= __expf(Gs[e % GC]);   // T diag(gamma beta)
  __syncthreads();
  for (int t = warp; t < 32; t += NW) {                                // dk = acc + Ab K + Ab^T K + (T diag(gamma beta))^T dW
    const int ti = t >> 3, tj = t & 7;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::load_matrix_sync(acc, tD + ti * 16 * LD4 + tj * 16, LD4, wm::mem_row_major);
    tile_mma<GC, false, false>(acc, Y1 + ti * 16 * LP, LP, tK + tj * 16, LD4);
    tile_mma<GC, true, false>(acc, Y1 + ti * 16, LP, tK + tj * 16, LD4);
    tile_mma<GC, true, false>(acc, Y3 + ti * 16, LP, tV + tj * 16, LD4);
    wm::store_matrix_sync(dk + vo + static_cast<long long>(ti) * 16 * ldv + tj * 16, acc, static_cast<unsigned>(ldv), wm::mem_row_major);
  }
  if (tid < GC) {
    const long long o = (static_cast<long long>(b) * d.T + c * GC + tid) * d.Hv + hv;
    dG[o] = dGs[tid];
    dbeta[o] = dbs[tid];
  }
}


template <bool BWD>
const char* launch_scan(const float* A1, const float* A2, const float* V0, const float* R0, const float* gl, const float* Rinit,
                        int B, int Hv, int n, float* Vout, float* Rchunks, float* Rfinal, cudaStream_t stream) {
  if (n > 1024) return "gdn_tc: at most 1024 chunks (65536 tokens) per sequence";
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // narrower column slices when the heads alone would leave SMs idle
  const bool narrow = static_cast<long long>(B) * Hv * 2 < sms;
  if (!FERRL_ONCE_PER_DEVICE(
          cudaFuncSetAttribute(gdn_scan_kernel<64, BWD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(ScanSmem<64>::BYTES)) == cudaSuccess &&
          cudaFuncSetAttribute(gdn_scan_kernel<32, BWD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(ScanSmem<32>::BYTES)) == cudaSuccess))
    return "gdn_tc: cannot reserve shared memory";
  if (narrow)
    gdn_scan_kernel<32, BWD><<<dim3(Hv * 4, B), kScanThreads, ScanSmem<32>::BYTES, stream>>>(A1, A2, V0, R0, gl, Rinit, n, 4, Vout, Rchunks,
                                                                                    Rfinal);
  else
    gdn_scan_kernel<64, BWD><<<dim3(Hv * 2, B), kScanThreads, ScanSmem<64>::BYTES, stream>>>(A1, A2, V0, R0, gl, Rinit, n, 2, Vout, Rchunks,
                                                                                    Rfinal);
  count_launch();
  return nullptr;
}

}  // namespace

const char* gdn_tc_forward(const float* q, const float* k, const float* v, const float* g, const float* beta, const float* S0,
                           int B, int T, int Hk, int Hv, float* Gc, float* gl, float* Tm, float* U, float* Wn, float* Kd,
                           float* out, float* S_out, float* Sin, float* Vn, cudaStream_t stream) {
  if (T % GC) return "gdn_tc: the sequence length must be a multiple of 64 (pad with beta = 0, g = 0)";
  if (Hk <= 0 || Hv % Hk) return "gdn_tc: value heads must be a multiple of key heads";
  if (B == 0 || T == 0) return nullptr;
  GdnDims d{B, T, Hk, Hv, T / GC};
  if (!FERRL_ONCE_PER_DEVICE(
          cudaFuncSetAttribute(gdn_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPrepSmem)) == cudaSuccess &&
          cudaFuncSetAttribute(gdn_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kOutSmem)) == cudaSuccess))
    return "gdn_tc: cannot reserve shared memory";
  gdn_prep_kernel<<<dim3(d.n, Hv, B), 256, kPrepSmem, stream>>>(k, v, g, beta, d, Gc, gl, Tm, U, Wn, Kd);
  count_launch();
  if (const char* e = launch_scan<false>(Wn, Kd, U, nullptr, gl, S0, B, Hv, d.n, Vn, Sin, S_out, stream)) return e;
  gdn_out_kernel<<<dim3(d.n, Hv, B), 512, kOutSmem, stream>>>(q, k, Gc, Sin, Vn, d, out);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_tc forward launch failed";
}

const char* gdn_tc_backward(const float* q, const float* k, const float* v, const float* beta, const float* Gc, const float* gl,
                            const float* Tm, const float* Wn, const float* Kd, const float* Vn, const float* Sin,
                            const float* dO, const float* dS_final, int B, int T, int Hk, int Hv, float* X0, float* Y0,
                            float* dVn, float* dSout, float* dW, float* dGpart, float* dq, float* dk, float* dv, float* dbeta,
                            float* dG, float* dS0, cudaStream_t stream) {
  if (T % GC) return "gdn_tc: the sequence length must be a multiple of 64";
  if (Hk <= 0 || Hv % Hk) return "gdn_tc: value heads must be a multiple of key heads";
  if (B == 0 || T == 0) return nullptr;
  GdnDims d{B, T, Hk, Hv, T / GC};
  if (!FERRL_ONCE_PER_DEVICE(
          cudaFuncSetAttribute(gdn_bwd_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kBwdPrepSmem)) == cudaSuccess &&
          cudaFuncSetAttribute(gdn_bwd_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kBwdStateSmem)) == cudaSuccess &&
          cudaFuncSetAttribute(gdn_bwd_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kBwdIntraSmem)) == cudaSuccess))
    return "gdn_tc: cannot reserve shared memory";
  gdn_bwd_prep_kernel<<<dim3(d.n, Hv, B), 512, kBwdPrepSmem, stream>>>(q, k, Gc, dO, d, X0, Y0);
  count_launch();
  if (const char* e = launch_scan<true>(Kd, Wn, X0, Y0, gl, dS_final, B, Hv, d.n, dVn, dSout, dS0, stream)) return e;
  gdn_bwd_state_kernel<<<dim3(d.n * 2, Hv, B), 256, kBwdStateSmem, stream>>>(q, k, Gc, Vn, dVn, Sin, dSout, dO, d, dq, dk, dW, dGpart);
  count_launch();
  gdn_bwd_intra_kernel<<<dim3(d.n, Hv, B), kIntraThreads, kBwdIntraSmem, stream>>>(q, k, v, beta, Gc, Tm, Vn, dVn, dW, dO, dGpart, d,
                                                                                 dq, dk, dv, dbeta, dG);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_tc backward launch failed";
}

}  // namespace ferrl
