// GatedDeltaNet kernels for sm_100a (Qwen3.5/3.6 linear-attention layers).
//
// Reference: crates/ferrl/src/gdn.rs - causal depthwise conv with left context :102-142, the
// single-step recurrent delta rule :286-317.  The reference composes both from tensor ops (a
// dozen launches per layer per token in decode); here each is one memory-bound kernel:
//
//   gdn_conv_fwd / gdn_conv_bwd  causal depthwise conv (+SiLU) over [B, L, C] without transposes,
//                                reading the K-1 tokens of left context from the carried state
//   gdn_conv_step                the one-token decode form; shifts the state in place
//   gdn_decode_step              L2-normalise q,k; S <- S*exp(g); delta rule update; o = S^T q,
//                                with the [kd, vd] fp32 state read and written exactly once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "../api.h"
#include "../common.cuh"

namespace ferrl {

namespace {

constexpr int kMaxConvK = 8;

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float dsilu_f(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// x [B, L, C] (row stride ldx), w [C, K], left [B, C, K-1] or null, y [B, L, C] contiguous.
// One thread per (b, t, c); consecutive threads walk c, so every access is coalesced.
__global__ void gdn_conv_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                                    const __nv_bfloat16* __restrict__ left, int B, int L, int C, int K, int act,
                                    __nv_bfloat16* __restrict__ y) {
  const long long n = static_cast<long long>(B) * L * C;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % C);
    const long long bt = i / C;
    const int t = static_cast<int>(bt % L), b = static_cast<int>(bt / L);
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
      const int ts = t - (K - 1) + j;
      float xv;
      if (ts >= 0) xv = __bfloat162float(x[(static_cast<long long>(b) * L + ts) * ldx + c]);
      else xv = left ? __bfloat162float(left[(static_cast<long long>(b) * C + c) * (K - 1) + (K - 1 + ts)]) : 0.f;
      acc += __bfloat162float(w[c * K + j]) * xv;
    }
    // the eager form rounds the conv output to the activation dtype before the SiLU
    acc = __bfloat162float(__float2bfloat16_rn(acc));
    y[i] = __float2bfloat16_rn(act ? silu_f(acc) : acc);
  }
}

// dx[b,t,c] = sum_j w[c,j] * dpre[b, t + K-1-j, c], dpre = dy * silu'(pre); pre is recomputed.
__global__ void gdn_conv_bwd_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                                    const __nv_bfloat16* __restrict__ left, const __nv_bfloat16* __restrict__ dy,
                                    int B, int L, int C, int K, int act, __nv_bfloat16* __restrict__ dx) {
  const long long n = static_cast<long long>(B) * L * C;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % C);
    const long long bt = i / C;
    const int t = static_cast<int>(bt % L), b = static_cast<int>(bt / L);
    float wv[kMaxConvK];
    for (int j = 0; j < K; ++j) wv[j] = __bfloat162float(w[c * K + j]);
    // inputs x[t-(K-1) .. t+(K-1)] cover every output this input feeds
    float xin[2 * kMaxConvK - 1];
    for (int o = 0; o < 2 * K - 1; ++o) {
      const int ts = t - (K - 1) + o;
      if (ts >= L) xin[o] = 0.f;
      else if (ts >= 0) xin[o] = __bfloat162float(x[(static_cast<long long>(b) * L + ts) * ldx + c]);
      else xin[o] = left ? __bfloat162float(left[(static_cast<long long>(b) * C + c) * (K - 1) + (K - 1 + ts)]) : 0.f;
    }
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
      const int to = t + (K - 1) - j;       // output position that reads x[t] through tap j
      if (to >= L) continue;
      float d = __bfloat162float(dy[(static_cast<long long>(b) * L + to) * C + c]);
      if (act) {
        float pre = 0.f;
        for (int jj = 0; jj < K; ++jj) pre += wv[jj] * xin[(to - t) + jj];
        pre = __bfloat162float(__float2bfloat16_rn(pre));
        d *= dsilu_f(pre);
      }
      acc += wv[j] * d;
    }
    dx[i] = __float2bfloat16_rn(acc);
  }
}

// One token: y[b,c] = act(sum_j w[c,j] * ctx[j]), ctx = [state[b,c,:], x[b,c]]; state shifts left.
__global__ void gdn_conv_step_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ state, int B, int C, int K, int act,
                                     __nv_bfloat16* __restrict__ y) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * C) return;
  const int c = i % C, b = i / C;
  __nv_bfloat16* st = state + static_cast<long long>(i) * (K - 1);
  const __nv_bfloat16 xv = x[static_cast<long long>(b) * ldx + c];
  float acc = __bfloat162float(w[c * K + K - 1]) * __bfloat162float(xv);
  for (int j = 0; j < K - 1; ++j) {
    const __nv_bfloat16 s = st[j];
    acc += __bfloat162float(w[c * K + j]) * __bfloat162float(s);
    if (j > 0) st[j - 1] = s;
  }
  if (K > 1) st[K - 2] = xv;
  acc = __bfloat162float(__float2bfloat16_rn(acc));
  y[i] = __float2bfloat16_rn(act ? silu_f(acc) : acc);
}

// One block per (b, value head); thread j owns column j of S [KD, VD] and keeps it in registers.
// q,k [B, Hk, KD] bf16 (row stride given), v [B, Hv, VD], g,beta [B, Hv] fp32, S [B, Hv, KD, VD] fp32.
template <int KD>
__global__ void gdn_decode_step_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                       const __nv_bfloat16* __restrict__ v, long long ldq, long long ldk, long long ldv,
                                       const float* __restrict__ g, const float* __restrict__ beta,
                                       float* __restrict__ S, int Hk, int Hv, int VD, int l2norm, float eps,
                                       __nv_bfloat16* __restrict__ out, GdnRawGates raw) {
  __shared__ float qs[KD], ks[KD], red[32];
  const int b = blockIdx.x / Hv, hv = blockIdx.x % Hv;
  const int hk = hv / (Hv / Hk);
  const int tid = threadIdx.x;
  float qq = 0.f, kk = 0.f;
  for (int i = tid; i < KD; i += blockDim.x) {
    const float qv = __bfloat162float(q[static_cast<long long>(b) * ldq + hk * KD + i]);
    const float kv = __bfloat162float(k[static_cast<long long>(b) * ldk + hk * KD + i]);
    qs[i] = qv;
    ks[i] = kv;
    qq += qv * qv;
    kk += kv * kv;
  }
  float qn = 1.f, kn = 1.f;
  if (l2norm) {
    qn = rsqrtf(block_sum(qq, red) + eps);
    kn = rsqrtf(block_sum(kk, red) + eps);
  }
  __syncthreads();
  const float qscale = qn * rsqrtf(static_cast<float>(KD));
  const long long bh = static_cast<long long>(b) * Hv + hv;
  float eg, bt;
  if (raw.a) {
    // gates from the projection output: g = -exp(A_log) softplus(a + dt_bias), beta = sigmoid(b)
    const float x = __bfloat162float(raw.a[static_cast<long long>(b) * raw.lda + hv]) + raw.dt_bias[hv];
    const float sp = x > 20.f ? x : log1pf(__expf(x));
    eg = __expf(-__expf(raw.A_log[hv]) * sp);
    bt = 1.f / (1.f + __expf(-__bfloat162float(raw.b[static_cast<long long>(b) * raw.ldb + hv])));
  } else {
    eg = __expf(g[bh]);
    bt = beta[bh];
  }
  for (int j = tid; j < VD; j += blockDim.x) {
    float* Sc = S + bh * KD * VD + j;
    float col[KD];
    float kv = 0.f;
#pragma unroll
    for (int i = 0; i < KD; ++i) {
      col[i] = Sc[static_cast<long long>(i) * VD] * eg;
      kv += col[i] * (ks[i] * kn);
    }
    const float delta = (__bfloat162float(v[static_cast<long long>(b) * ldv + hv * VD + j]) - kv) * bt;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < KD; ++i) {
      col[i] += (ks[i] * kn) * delta;
      o += col[i] * (qs[i] * qscale);
      Sc[static_cast<long long>(i) * VD] = col[i];
    }
    out[bh * VD + j] = __float2bfloat16_rn(o);
  }
}

// The same step for KD x VD states that divide over 256 threads: thread (row group, column group) keeps RPT rows x 4
// columns of S in registers (16 x float4 at 128 x 128), so every load and store is a 16-byte access of a 512-byte row
// and all of a CTA's 64 KB are in flight at once; the two dot products (S^T k and S^T q) are finished across the row
// groups through shared memory in a fixed order.  (One column per thread, as above, needs KD registers per thread and
// spills at KD = 128.)
template <int KD, int VD>
__global__ void __launch_bounds__(256)
gdn_decode_step_tile_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                            const __nv_bfloat16* __restrict__ v, long long ldq, long long ldk, long long ldv,
                            const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ S, int Hk,
                            int Hv, int l2norm, float eps, __nv_bfloat16* __restrict__ out, GdnRawGates raw) {
  constexpr int CG = VD / 4, RG = 256 / CG, RPT = KD / RG;
  static_assert(VD % 4 == 0 && 256 % CG == 0 && KD % RG == 0 && RPT >= 1, "state does not divide over 256 threads");
  __shared__ float qs[KD], ks[KD], red[32];
  __shared__ __align__(16) float part[RG][VD];
  const int b = blockIdx.x / Hv, hv = blockIdx.x % Hv;
  const int hk = hv / (Hv / Hk);
  const int tid = threadIdx.x;
  const int cg = tid % CG, rg = tid / CG;
  const long long bh = static_cast<long long>(b) * Hv + hv;
  // the state does not depend on anything computed here: request it first
  float4* Sp = reinterpret_cast<float4*>(S + bh * KD * VD) + static_cast<long long>(rg) * RPT * CG + cg;
  float4 col[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) col[i] = Sp[i * CG];
  float qq = 0.f, kk = 0.f;
  for (int i = tid; i < KD; i += 256) {
    const float qv = __bfloat162float(q[static_cast<long long>(b) * ldq + hk * KD + i]);
    const float kv = __bfloat162float(k[static_cast<long long>(b) * ldk + hk * KD + i]);
    qs[i] = qv;
    ks[i] = kv;
    qq += qv * qv;
    kk += kv * kv;
  }
  float qn = 1.f, kn = 1.f;
  if (l2norm) {
    qn = rsqrtf(block_sum(qq, red) + eps);
    kn = rsqrtf(block_sum(kk, red) + eps);
  }
  __syncthreads();
  const float qscale = qn * rsqrtf(static_cast<float>(KD));
  float eg, bt;
  if (raw.a) {
    const float x = __bfloat162float(raw.a[static_cast<long long>(b) * raw.lda + hv]) + raw.dt_bias[hv];
    const float sp = x > 20.f ? x : log1pf(__expf(x));
    eg = __expf(-__expf(raw.A_log[hv]) * sp);
    bt = 1.f / (1.f + __expf(-__bfloat162float(raw.b[static_cast<long long>(b) * raw.ldb + hv])));
  } else {
    eg = __expf(g[bh]);
    bt = beta[bh];
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const float kx = ks[rg * RPT + i] * kn;
    col[i].x *= eg; col[i].y *= eg; col[i].z *= eg; col[i].w *= eg;
    acc.x += col[i].x * kx; acc.y += col[i].y * kx; acc.z += col[i].z * kx; acc.w += col[i].w * kx;
  }
  *reinterpret_cast<float4*>(&part[rg][cg * 4]) = acc;
  __syncthreads();
  float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int r = 0; r < RG; ++r) {
    const float4 t = *reinterpret_cast<const float4*>(&part[r][cg * 4]);
    kv.x += t.x; kv.y += t.y; kv.z += t.z; kv.w += t.w;
  }
  const __nv_bfloat16* vp = v + static_cast<long long>(b) * ldv + hv * VD + cg * 4;
  float4 delta;
  delta.x = (__bfloat162float(vp[0]) - kv.x) * bt;
  delta.y = (__bfloat162float(vp[1]) - kv.y) * bt;
  delta.z = (__bfloat162float(vp[2]) - kv.z) * bt;
  delta.w = (__bfloat162float(vp[3]) - kv.w) * bt;
  acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const float kx = ks[rg * RPT + i] * kn, qx = qs[rg * RPT + i] * qscale;
    col[i].x += kx * delta.x; col[i].y += kx * delta.y; col[i].z += kx * delta.z; col[i].w += kx * delta.w;
    acc.x += col[i].x * qx; acc.y += col[i].y * qx; acc.z += col[i].z * qx; acc.w += col[i].w * qx;
    Sp[i * CG] = col[i];
  }
  __syncthreads();                       // every thread has read the first sums
  *reinterpret_cast<float4*>(&part[rg][cg * 4]) = acc;
  __syncthreads();
  if (tid < VD) {
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < RG; ++r) o += part[r][tid];
    out[bh * VD + tid] = __float2bfloat16_rn(o);
  }
}

// ------------------------------------------------------------------------------------------------
// Chunked gated delta rule, forward (crates/ferrl/src/gdn.rs:451-556 composes it from ~40 tensor
// ops per chunk).  One CTA per (batch row, value head) walks the sequence in chunks of 64 tokens
// with the [128, 128] fp32 state resident in shared memory the whole time:
//
//   1. load q,k (L2-normalised, q scaled), v*beta, cumulative log-decay G, k*beta*exp(G)
//   2. A = tril(beta_i exp(G_i-G_j) <k_i,k_j>, -1)
//   3. (I + A) [u | w] = [v*beta | k*beta*exp(G)] by forward substitution, one column per thread
//      held in registers (the unit-triangular solve the reference does in 8x8 blocks)
//   4. v_new = u - w S
//   5. P = tril(exp(G_i-G_j) <q_i,k_j>)
//   6. o = (q exp(G)) S + P v_new
//   7. S <- S exp(G_last) + (k exp(G_last-G))^T v_new
//
// All products are fp32 FMAs on register micro-tiles (4x4, 4x8, 8x8) fed from shared memory; the
// arithmetic and its order inside a chunk are fixed, so results are bit-reproducible.
constexpr int GC = 64;      // chunk length
constexpr int GD = 128;     // key and value head dim of this kernel

__global__ void __launch_bounds__(256, 1)
gdn_chunk_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                     const __nv_bfloat16* __restrict__ v, long long q_bs, long long q_ts, long long k_bs,
                     long long k_ts, long long v_bs, long long v_ts, const float* __restrict__ g,
                     const float* __restrict__ beta, const float* __restrict__ S0, float* __restrict__ S_out,
                     __nv_bfloat16* __restrict__ out, int T, int Hk, int Hv, int l2norm, float eps) {
  extern __shared__ __align__(16) float gsm[];
  float* S = gsm;                     // [GD][GD]
  float* ks = S + GD * GD;            // [GC][GD]
  float* qs = ks + GC * GD;           // [GC][GD]
  float* us = qs + GC * GD;           // [GC][GD]  v*beta -> u -> v_new
  float* ws = us + GC * GD;           // [GC][GD]  k*beta*exp(G) -> w
  float* A = ws + GC * GD;            // [GC][GC]
  float* Gc = A + GC * GC;            // [GC] cumulative log decay
  float* bt = Gc + GC;                // [GC]
  const int b = blockIdx.x / Hv, hv = blockIdx.x % Hv;
  const int hk = hv / (Hv / Hk);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long bh = static_cast<long long>(b) * Hv + hv;
  const float qscale = rsqrtf(static_cast<float>(GD));

  for (int i = tid; i < GD * GD; i += 256) S[i] = S0 ? S0[bh * GD * GD + i] : 0.f;

  for (int c0 = 0; c0 < T; c0 += GC) {
    const int n = min(GC, T - c0);
    __syncthreads();
    // ---- 1. loads
    if (tid < GC) {
      const long long gi = (static_cast<long long>(b) * T + c0 + tid) * Hv + hv;
      Gc[tid] = tid < n ? g[gi] : 0.f;
      bt[tid] = tid < n ? beta[gi] : 0.f;
    }
    __syncthreads();
    if (tid == 0) {
      float acc = 0.f;
      for (int i = 0; i < GC; ++i) {
        acc += Gc[i];
        Gc[i] = acc;
      }
    }
    for (int r = warp; r < GC; r += 8) {       // a warp per row, 4 channels per lane
      float kv[4] = {0.f, 0.f, 0.f, 0.f}, qv[4] = {0.f, 0.f, 0.f, 0.f}, vv[4] = {0.f, 0.f, 0.f, 0.f};
      if (r < n) {
        const __nv_bfloat16* kp = k + b * k_bs + (c0 + r) * k_ts + hk * GD + lane * 4;
        const __nv_bfloat16* qp = q + b * q_bs + (c0 + r) * q_ts + hk * GD + lane * 4;
        const __nv_bfloat16* vp = v + b * v_bs + (c0 + r) * v_ts + hv * GD + lane * 4;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          kv[e] = __bfloat162float(kp[e]);
          qv[e] = __bfloat162float(qp[e]);
          vv[e] = __bfloat162float(vp[e]);
        }
      }
      float kn = 1.f, qn = 1.f;
      if (l2norm) {
        kn = rsqrtf(warp_sum(kv[0] * kv[0] + kv[1] * kv[1] + kv[2] * kv[2] + kv[3] * kv[3]) + eps);
        qn = rsqrtf(warp_sum(qv[0] * qv[0] + qv[1] * qv[1] + qv[2] * qv[2] + qv[3] * qv[3]) + eps);
      }
      *reinterpret_cast<float4*>(ks + r * GD + lane * 4) = make_float4(kv[0] * kn, kv[1] * kn, kv[2] * kn, kv[3] * kn);
      const float qm = qn * qscale;
      *reinterpret_cast<float4*>(qs + r * GD + lane * 4) = make_float4(qv[0] * qm, qv[1] * qm, qv[2] * qm, qv[3] * qm);
      *reinterpret_cast<float4*>(us + r * GD + lane * 4) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    }
    __syncthreads();
    for (int i = tid; i < GC * GD; i += 256) {
      const int r = i / GD;
      us[i] *= bt[r];
      ws[i] = ks[i] * bt[r] * __expf(Gc[r]);
    }
    // ---- 2. A = strictly lower part of beta_i exp(G_i-G_j) <k_i,k_j>; 4x4 tile per thread
    {
      const int ti = tid / 16, tj = tid % 16;
      float acc[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;
      if (tj <= ti) {
        for (int dd = 0; dd < GD; ++dd) {
          const int d = (dd + lane) & (GD - 1);    // each lane starts at its own channel: no bank conflicts
          float ka[4], kb[4];
#pragma unroll
          for (int a = 0; a < 4; ++a) {
            ka[a] = ks[(4 * ti + a) * GD + d];
            kb[a] = ks[(4 * tj + a) * GD + d];
          }
#pragma unroll
          for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][c] += ka[a] * kb[c];
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int i = 4 * ti + a, j = 4 * tj + c;
          A[i * GC + j] = (j < i) ? acc[a][c] * bt[i] * __expf(Gc[i] - Gc[j]) : 0.f;
        }
    }
    __syncthreads();
    // ---- 3. forward substitution; thread t owns column t of [u | w]
    {
      float* col = (tid < GD) ? (us + tid) : (ws + (tid - GD));
      float x[GC];
#pragma unroll
      for (int i = 0; i < GC; ++i) x[i] = col[i * GD];
#pragma unroll
      for (int i = 1; i < GC; ++i) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < i; ++j) acc += A[i * GC + j] * x[j];
        x[i] -= acc;
      }
#pragma unroll
      for (int i = 0; i < GC; ++i) col[i * GD] = x[i];
    }
    __syncthreads();
    // ---- 4. v_new = u - w S; 4 rows x 8 cols per thread
    const int tr = tid / 16, tc = tid % 16;
    {
      float acc[4][8];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[a][c] = 0.f;
      for (int d = 0; d < GD; ++d) {
        const float4 s0 = *reinterpret_cast<const float4*>(S + d * GD + tc * 8);
        const float4 s1 = *reinterpret_cast<const float4*>(S + d * GD + tc * 8 + 4);
        const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const float wv = ws[(4 * tr + a) * GD + d];
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[a][c] += wv * sv[c];
        }
      }
      __syncthreads();     // everyone has finished reading ws/us of this phase's inputs before us changes
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 8; ++c) us[(4 * tr + a) * GD + tc * 8 + c] -= acc[a][c];
    }
    // ---- 5. P = lower (inclusive) part of exp(G_i-G_j) <q_i,k_j>, into A (L is no longer needed)
    {
      const int ti = tid / 16, tj = tid % 16;
      float acc[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;
      if (tj <= ti) {
        for (int dd = 0; dd < GD; ++dd) {
          const int d = (dd + lane) & (GD - 1);
          float qa[4], kb[4];
#pragma unroll
          for (int a = 0; a < 4; ++a) {
            qa[a] = qs[(4 * ti + a) * GD + d];
            kb[a] = ks[(4 * tj + a) * GD + d];
          }
#pragma unroll
          for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][c] += qa[a] * kb[c];
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int i = 4 * ti + a, j = 4 * tj + c;
          A[i * GC + j] = (j <= i) ? acc[a][c] * __expf(Gc[i] - Gc[j]) : 0.f;
        }
    }
    __syncthreads();
    // ---- 6. o = (q exp(G)) S + P v_new
    {
      float acc[4][8];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[a][c] = 0.f;
      float eg[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) eg[a] = __expf(Gc[4 * tr + a]);
      for (int d = 0; d < GD; ++d) {
        const float4 s0 = *reinterpret_cast<const float4*>(S + d * GD + tc * 8);
        const float4 s1 = *reinterpret_cast<const float4*>(S + d * GD + tc * 8 + 4);
        const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const float qv = qs[(4 * tr + a) * GD + d] * eg[a];
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[a][c] += qv * sv[c];
        }
      }
      for (int j = 0; j < GC; ++j) {
        const float4 u0 = *reinterpret_cast<const float4*>(us + j * GD + tc * 8);
        const float4 u1 = *reinterpret_cast<const float4*>(us + j * GD + tc * 8 + 4);
        const float uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const float pv = A[(4 * tr + a) * GC + j];
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[a][c] += pv * uv[c];
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int r = 4 * tr + a;
        if (r < n) {
          uint4 o;
          __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int c = 0; c < 4; ++c) oh[c] = __floats2bfloat162_rn(acc[a][2 * c], acc[a][2 * c + 1]);
          *reinterpret_cast<uint4*>(out + ((static_cast<long long>(b) * T + c0 + r) * Hv + hv) * GD + tc * 8) = o;
        }
      }
    }
    __syncthreads();
    // ---- 7. S <- S exp(G_last) + (k exp(G_last - G))^T v_new; 8x8 tile per thread
    {
      const float glast = Gc[GC - 1];
      const float eglast = __expf(glast);
      const int td = tid / 16, tcc = tid % 16;
      float acc[8][8];
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        const float4 s0 = *reinterpret_cast<const float4*>(S + (8 * td + a) * GD + tcc * 8);
        const float4 s1 = *reinterpret_cast<const float4*>(S + (8 * td + a) * GD + tcc * 8 + 4);
        acc[a][0] = s0.x * eglast; acc[a][1] = s0.y * eglast; acc[a][2] = s0.z * eglast; acc[a][3] = s0.w * eglast;
        acc[a][4] = s1.x * eglast; acc[a][5] = s1.y * eglast; acc[a][6] = s1.z * eglast; acc[a][7] = s1.w * eglast;
      }
      for (int i = 0; i < GC; ++i) {
        const float dec = __expf(glast - Gc[i]);
        const float4 k0 = *reinterpret_cast<const float4*>(ks + i * GD + td * 8);
        const float4 k1 = *reinterpret_cast<const float4*>(ks + i * GD + td * 8 + 4);
        const float4 u0 = *reinterpret_cast<const float4*>(us + i * GD + tcc * 8);
        const float4 u1 = *reinterpret_cast<const float4*>(us + i * GD + tcc * 8 + 4);
        const float kv[8] = {k0.x * dec, k0.y * dec, k0.z * dec, k0.w * dec, k1.x * dec, k1.y * dec, k1.z * dec, k1.w * dec};
        const float uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
        for (int a = 0; a < 8; ++a)
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[a][c] += kv[a] * uv[c];
      }
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        *reinterpret_cast<float4*>(S + (8 * td + a) * GD + tcc * 8) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
        *reinterpret_cast<float4*>(S + (8 * td + a) * GD + tcc * 8 + 4) = make_float4(acc[a][4], acc[a][5], acc[a][6], acc[a][7]);
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < GD * GD; i += 256) S_out[bh * GD * GD + i] = S[i];
}

}  // namespace

const char* gdn_conv_fwd(const void* x, long long ldx, const void* w, const void* left, int B, int L, int C, int K,
                         bool act, void* y, cudaStream_t stream) {
  if (K < 1 || K > kMaxConvK) return "gdn_conv: kernel width 1..8";
  const long long n = static_cast<long long>(B) * L * C;
  if (n == 0) return nullptr;
  const int blocks = static_cast<int>(std::min<long long>((n + 255) / 256, 148 * 32));
  gdn_conv_fwd_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ldx,
                                                  static_cast<const __nv_bfloat16*>(w),
                                                  static_cast<const __nv_bfloat16*>(left), B, L, C, K, act ? 1 : 0,
                                                  static_cast<__nv_bfloat16*>(y));
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_conv_fwd launch failed";
}

const char* gdn_conv_bwd(const void* x, long long ldx, const void* w, const void* left, const void* dy, int B, int L,
                         int C, int K, bool act, void* dx, cudaStream_t stream) {
  if (K < 1 || K > kMaxConvK) return "gdn_conv: kernel width 1..8";
  const long long n = static_cast<long long>(B) * L * C;
  if (n == 0) return nullptr;
  const int blocks = static_cast<int>(std::min<long long>((n + 255) / 256, 148 * 32));
  gdn_conv_bwd_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ldx,
                                                  static_cast<const __nv_bfloat16*>(w),
                                                  static_cast<const __nv_bfloat16*>(left),
                                                  static_cast<const __nv_bfloat16*>(dy), B, L, C, K, act ? 1 : 0,
                                                  static_cast<__nv_bfloat16*>(dx));
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_conv_bwd launch failed";
}

const char* gdn_conv_step(const void* x, long long ldx, const void* w, void* state, int B, int C, int K, bool act,
                          void* y, cudaStream_t stream) {
  if (K < 1 || K > kMaxConvK) return "gdn_conv: kernel width 1..8";
  if (B * C == 0) return nullptr;
  gdn_conv_step_kernel<<<(B * C + 255) / 256, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ldx,
                                                                static_cast<const __nv_bfloat16*>(w),
                                                                static_cast<__nv_bfloat16*>(state), B, C, K, act ? 1 : 0,
                                                                static_cast<__nv_bfloat16*>(y));
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_conv_step launch failed";
}

const char* gdn_chunk_fwd(const void* q, const void* k, const void* v, long long q_bs, long long q_ts, long long k_bs,
                          long long k_ts, long long v_bs, long long v_ts, const float* g, const float* beta,
                          const float* S0, float* S_out, void* out, int B, int T, int Hk, int Hv, int KD, int VD,
                          bool l2norm, float eps, cudaStream_t stream) {
  if (KD != GD || VD != GD) return "gdn_chunk_fwd: key and value head dim must be 128";
  if (Hk <= 0 || Hv % Hk) return "gdn_chunk_fwd: value heads must be a multiple of key heads";
  if (B == 0 || T == 0) return nullptr;
  constexpr size_t smem = (static_cast<size_t>(GD) * GD + 4 * GC * GD + GC * GC + 2 * GC) * sizeof(float);
  if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(gdn_chunk_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  static_cast<int>(smem)) == cudaSuccess))
    return "gdn_chunk_fwd: cannot reserve shared memory";
  gdn_chunk_fwd_kernel<<<B * Hv, 256, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      q_bs, q_ts, k_bs, k_ts, v_bs, v_ts, g, beta, S0, S_out, static_cast<__nv_bfloat16*>(out), T, Hk, Hv,
      l2norm ? 1 : 0, eps);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_chunk_fwd launch failed";
}

const char* gdn_decode_step(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv,
                            const float* g, const float* beta, float* S, int B, int Hk, int Hv, int KD, int VD,
                            bool l2norm, float eps, void* out, cudaStream_t stream, const GdnRawGates* raw_gates) {
  if (Hk <= 0 || Hv % Hk) return "gdn_decode_step: value heads must be a multiple of key heads";
  GdnRawGates raw{};
  if (raw_gates) raw = *raw_gates;
  if (!raw.a && (!g || !beta)) return "gdn_decode_step: either g and beta or the raw gate inputs are needed";
  if (raw.a && (!raw.b || !raw.A_log || !raw.dt_bias)) return "gdn_decode_step: incomplete raw gate inputs";
  if (B == 0) return nullptr;
  if (KD == 128 && VD == 128) {
    gdn_decode_step_tile_kernel<128, 128><<<B * Hv, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
        ldq, ldk, ldv, g, beta, S, Hk, Hv, l2norm ? 1 : 0, eps, static_cast<__nv_bfloat16*>(out), raw);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_decode_step launch failed";
  }
  const int threads = std::min(256, (VD + 31) / 32 * 32);
#define FERRL_GDN_STEP(KDV)                                                                                        \
  gdn_decode_step_kernel<KDV><<<B * Hv, threads, 0, stream>>>(                                                     \
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), \
      ldq, ldk, ldv, g, beta, S, Hk, Hv, VD, l2norm ? 1 : 0, eps, static_cast<__nv_bfloat16*>(out), raw)
  switch (KD) {
    case 16: FERRL_GDN_STEP(16); break;
    case 32: FERRL_GDN_STEP(32); break;
    case 64: FERRL_GDN_STEP(64); break;
    case 128: FERRL_GDN_STEP(128); break;
    default: return "gdn_decode_step: key dim must be 16, 32, 64 or 128";
  }
#undef FERRL_GDN_STEP
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "gdn_decode_step launch failed";
}

}  // namespace ferrl
