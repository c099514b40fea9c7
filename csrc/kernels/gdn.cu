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
                                       __nv_bfloat16* __restrict__ out) {
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
  const float eg = __expf(g[bh]);
  const float bt = beta[bh];
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

const char* gdn_decode_step(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv,
                            const float* g, const float* beta, float* S, int B, int Hk, int Hv, int KD, int VD,
                            bool l2norm, float eps, void* out, cudaStream_t stream) {
  if (Hk <= 0 || Hv % Hk) return "gdn_decode_step: value heads must be a multiple of key heads";
  if (B == 0) return nullptr;
  const int threads = std::min(256, (VD + 31) / 32 * 32);
#define FERRL_GDN_STEP(KDV)                                                                                        \
  gdn_decode_step_kernel<KDV><<<B * Hv, threads, 0, stream>>>(                                                     \
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), \
      ldq, ldk, ldv, g, beta, S, Hk, Hv, VD, l2norm ? 1 : 0, eps, static_cast<__nv_bfloat16*>(out))
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
