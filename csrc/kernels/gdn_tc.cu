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
//   gdn_chunk_bwd_kernel  everything that does not cross chunks: dq, dk, dv, dbeta and dG (the caller turns
//                         dG into dg with a reverse cumulative sum inside each chunk)
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
// A points at the tile's first row (AT: first column of the stored [K, M] matrix), B likewise.
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
#pragma unroll
    for (int e = 0; e < a.num_elements; ++e) a.x[e] = wm::__float_to_tf32(a.x[e]);
#pragma unroll
    for (int e = 0; e < b.num_elements; ++e) b.x[e] = wm::__float_to_tf32(b.x[e]);
    wm::mma_sync(c, a, b, c);
  }
}

// ---------------------------------------------------------------------------------------------
// prep: per chunk G, T, U, Wn = -W, Kd = diag(exp(G_C - G)) K and gl = G_C.
// Shared: three [64, 64] matrices and two vectors.
__global__ void __launch_bounds__(256)
gdn_prep_kernel(const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ g,
                const float* __restrict__ beta, GdnDims d, float* __restrict__ Gc, float* __restrict__ gl,
                float* __restrict__ Tm, float* __restrict__ U, float* __restrict__ Wn, float* __restrict__ Kd) {
  extern __shared__ __align__(128) float sm[];
  float* Y1 = sm;                  // K K^T, then A
  float* Y2 = Y1 + GC * GC;        // T
  float* Y3 = Y2 + GC * GC;        // T diag(beta), then -T diag(gamma beta)
  float* Gs = Y3 + GC * GC;
  float* bs = Gs + GC;
  const int c = blockIdx.x, hv = blockIdx.y, b = blockIdx.z;
  const int hk = hv / (d.Hv / d.Hk);
  const int tid = threadIdx.x;
  const long long ldk = static_cast<long long>(d.Hk) * GD, ldv = static_cast<long long>(d.Hv) * GD;
  const float* kg = k + qk_off(d, b, c * GC, hk);
  const float* vg = v + v_off(d, b, c * GC, hv);
  const long long co = ch_off(d, b, hv, c);
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
  mm<false, true, false>(Y1, GC, kg, ldk, kg, ldk, GC, GC, GD);
  __syncthreads();
  const float glast = Gs[GC - 1];
  for (int e = tid; e < GC * GC; e += 256) {
    const int i = e / GC, j = e - i * GC;
    Y1[e] = (i > j) ? bs[i] * Y1[e] * __expf(Gs[i] - Gs[j]) : 0.f;
    Y2[e] = (i == j) ? 1.f : 0.f;
  }
  // Kd = diag(exp(G_C - G)) K, straight from global to global
  for (int e = tid; e < GC * GD / 4; e += 256) {
    const int i = e / (GD / 4), x = e - i * (GD / 4);
    float4 t = reinterpret_cast<const float4*>(kg + i * ldk)[x];
    const float f = __expf(glast - Gs[i]);
    reinterpret_cast<float4*>(Kd + co * GC * GD)[e] = make_float4(t.x * f, t.y * f, t.z * f, t.w * f);
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
  for (int e = tid; e < GC * GC; e += 256) {
    const int j = e % GC;
    Tm[co * GC * GC + e] = Y2[e];
    Y3[e] = Y2[e] * bs[j];
  }
  if (tid < GC) Gc[co * GC + tid] = Gs[tid];
  if (tid == 0) gl[co] = glast;
  __syncthreads();
  mm<false, false, false>(U + co * GC * GD, GD, Y3, GC, vg, ldv, GC, GD, GC);
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int j = e % GC;
    Y3[e] = -Y2[e] * bs[j] * __expf(Gs[j]);
  }
  __syncthreads();
  mm<false, false, false>(Wn + co * GC * GD, GD, Y3, GC, kg, ldk, GC, GD, GC);
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

template <int DV, bool BWD>
__global__ void __launch_bounds__(256, 1)
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
  for (int e = tid; e < n; e += 256) gls[e] = gl[cbase + e];
  for (int e = tid; e < GD * DV; e += 256) {
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
    for (int e = tid; e < GD * DV; e += 256) {
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
    for (int t = warp; t < (GC / 16) * TN; t += 8) {
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
    float* rdst = last ? Rfinal : Rchunks + (cbase + c + step) * GD * GD;
    for (int t = warp; t < (GD / 16) * TN; t += 8) {
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

__global__ void __launch_bounds__(256, 1)
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
  for (int t = warp; t < 16; t += 8) {                 // P = Q K^T
    const int ti = t >> 2, tj = t & 3;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GD, false, true>(acc, Qs + ti * 16 * LD4, LD4, Ks + tj * 16 * LD4, LD4);
    wm::store_matrix_sync(P + ti * 16 * LP + tj * 16, acc, LP, wm::mem_row_major);
  }
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int i = e / GC, j = e - i * GC;
    P[i * LP + j] = (i >= j) ? P[i * LP + j] * __expf(Gs[i] - Gs[j]) : 0.f;
  }
  for (int e = tid; e < GC * GD; e += 256) {
    const int i = e / GD, x = e - i * GD;
    Qs[i * LD4 + x] *= __expf(Gs[i]);
  }
  cp_async_wait_all();
  __syncthreads();
  float* og = out + v_off(d, b, c * GC, hv);
  for (int t = warp; t < 32; t += 8) {                 // O = (gamma Q) Sin + P Vn
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

__global__ void __launch_bounds__(256, 1)
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
  for (int t = warp; t < 16; t += 8) {
    const int ti = t >> 2, tj = t & 3;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GD, false, true>(acc, Qs + ti * 16 * LD4, LD4, Ks + tj * 16 * LD4, LD4);
    wm::store_matrix_sync(P + ti * 16 * LP8 + tj * 16, acc, LP8, wm::mem_row_major);
  }
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int i = e / GC, j = e - i * GC;
    P[i * LP8 + j] = (i >= j) ? P[i * LP8 + j] * __expf(Gs[i] - Gs[j]) : 0.f;
  }
  for (int e = tid; e < GC * GD; e += 256) {
    const int i = e / GD, x = e - i * GD;
    Qs[i * LD4 + x] *= __expf(Gs[i]);
  }
  __syncthreads();
  for (int t = warp; t < 32; t += 8) {                 // X0 = P^T dO
    const int ti = t >> 3, tj = t & 7;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GC, true, false>(acc, P + ti * 16, LP8, Os + tj * 16, LD8);
    wm::store_matrix_sync(X0 + co * GC * GD + ti * 16 * GD + tj * 16, acc, GD, wm::mem_row_major);
  }
  for (int t = warp; t < 64; t += 8) {                 // Y0 = (gamma Q)^T dO
    const int ti = t >> 3, tj = t & 7;
    wm::fragment<wm::accumulator, 16, 16, 8, float> acc;
    wm::fill_fragment(acc, 0.f);
    tile_mma<GC, true, false>(acc, Qs + ti * 16, LD4, Os + tj * 16, LD8);
    wm::store_matrix_sync(Y0 + co * GD * GD + ti * 16 * GD + tj * 16, acc, GD, wm::mem_row_major);
  }
}

// ---------------------------------------------------------------------------------------------
// everything of the backward that stays inside a chunk.  Shared: E1, E2, E3 [64,128]; Y1, Y2, Y3
// [64,64]; vectors.  Operands that are plain inputs (q, k, v, dO, Vn, dVn, T, Sin, dSout) are read
// by the tensor-core loads straight from global memory.

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
  float* Rv = dbs + GC;           // [64]
  float* red = Rv + GC;           // [32]
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
    Rv[tid] = r;
  }
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
    for (int i = 0; i < GC; ++i) t += Rv[i];
    dGs[GC - 1] += t;
  }
  for (int e = tid; e < GC * GD; e += 256) E2[e] *= __expf(glast - Gs[e / GD]);
  __syncthreads();
  mm<true, false, true>(E2, GD, Y1, GC, qg, ldk, GC, GD, GC);
  // ---- gamma_C <Sin, dS'> goes to dG of the last row
  {
    float part = 0.f;
    for (int e = tid; e < GD * GD; e += 256) part += Sg[e] * dSg[e];
    const float tot = block_sum(part, red);
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
  mm<false, true, false>(Y1, GC, kg, ldk, kg, ldk, GC, GC, GD);        // K K^T (dT is no longer needed)
  __syncthreads();
  for (int e = tid; e < GC * GC; e += 256) {
    const int i = e / GC, j = e - i * GC;
    const float dad = (i > j) ? -Y3[e] * __expf(Gs[i] - Gs[j]) : 0.f;
    Y2[e] = dad * bs[i] * Y1[e];       // M_A = dA o A
    Y1[e] = dad;                       // dA o D
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
    dGs[tid] += rs - cs + __expf(Gs[tid]) * bs[tid] * t;
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
constexpr size_t kChunkBwdSmem = (3 * GC * GD + 3 * GC * GC + 5 * GC + 32) * sizeof(float);

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
    gdn_scan_kernel<32, BWD><<<dim3(Hv * 4, B), 256, ScanSmem<32>::BYTES, stream>>>(A1, A2, V0, R0, gl, Rinit, n, 4, Vout, Rchunks,
                                                                                    Rfinal);
  else
    gdn_scan_kernel<64, BWD><<<dim3(Hv * 2, B), 256, ScanSmem<64>::BYTES, stream>>>(A1, A2, V0, R0, gl, Rinit, n, 2, Vout, Rchunks,
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
  gdn_out_kernel<<<dim3(d.n, Hv, B), 256, kOutSmem, stream>>>(q, k, Gc, Sin, Vn, d, out);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_tc forward launch failed";
}

const char* gdn_tc_backward(const float* q, const float* k, const float* v, const float* beta, const float* Gc, const float* gl,
                            const float* Tm, const float* Wn, const float* Kd, const float* Vn, const float* Sin,
                            const float* dO, const float* dS_final, int B, int T, int Hk, int Hv, float* X0, float* Y0,
                            float* dVn, float* dSout, float* dq, float* dk, float* dv, float* dbeta, float* dG, float* dS0,
                            cudaStream_t stream) {
  if (T % GC) return "gdn_tc: the sequence length must be a multiple of 64";
  if (Hk <= 0 || Hv % Hk) return "gdn_tc: value heads must be a multiple of key heads";
  if (B == 0 || T == 0) return nullptr;
  GdnDims d{B, T, Hk, Hv, T / GC};
  if (!FERRL_ONCE_PER_DEVICE(
          cudaFuncSetAttribute(gdn_bwd_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kBwdPrepSmem)) == cudaSuccess &&
          cudaFuncSetAttribute(gdn_chunk_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kChunkBwdSmem)) == cudaSuccess))
    return "gdn_tc: cannot reserve shared memory";
  gdn_bwd_prep_kernel<<<dim3(d.n, Hv, B), 256, kBwdPrepSmem, stream>>>(q, k, Gc, dO, d, X0, Y0);
  count_launch();
  if (const char* e = launch_scan<true>(Kd, Wn, X0, Y0, gl, dS_final, B, Hv, d.n, dVn, dSout, dS0, stream)) return e;
  gdn_chunk_bwd_kernel<<<dim3(d.n, Hv, B), 256, kChunkBwdSmem, stream>>>(q, k, v, beta, Gc, Tm, Vn, dVn, Sin, dSout, dO, d, dq,
                                                                         dk, dv, dbeta, dG);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_tc backward launch failed";
}

}  // namespace ferrl
