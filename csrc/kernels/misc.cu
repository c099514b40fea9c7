// Small bandwidth-bound kernels: gated activation (SwiGLU / GeGLU) forward+backward,
// embedding gather, LoRA merge W + B*A, fused multi-tensor AdamW with global-norm clip,
// GRPO loss forward/backward.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"

namespace ferrl {
namespace {

__device__ __forceinline__ float act_fwd(float g, int act) {
  if (act == kActSilu) return g / (1.f + __expf(-g));
  // gelu tanh approximation
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float t = tanhf(k0 * (g + k1 * g * g * g));
  return 0.5f * g * (1.f + t);
}
__device__ __forceinline__ float act_grad(float g, int act) {
  if (act == kActSilu) {
    float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (g + k1 * g * g * g);
  float t = tanhf(u);
  float du = k0 * (1.f + 3.f * k1 * g * g);
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * du;
}

// gate_up [rows, 2F] laid out [gate | up] -> out [rows, F]
template <typename T>
__global__ void glu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows, int F, int act) {
  pdl_trigger();   // a dependent GEMM may start streaming its weights while this kernel runs
  pdl_wait();      // launched as a programmatic dependent itself: nothing is read before the predecessor is done
  long long n = rows * F;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long r = i / F;
    int c = static_cast<int>(i - r * F);
    float g = to_f(gu[r * 2 * F + c]);
    float u = to_f(gu[r * 2 * F + F + c]);
    out[i] = from_f<T>(act_fwd(g, act) * u);
  }
}
// bf16 vector forms: 8 elements per thread per step, 16-byte loads and stores; F % 8 == 0
__global__ void glu_fwd_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long rows,
                                   int F, int act) {
  pdl_trigger();   // a dependent GEMM may start streaming its weights while this kernel runs
  pdl_wait();      // launched as a programmatic dependent itself: nothing is read before the predecessor is done
  const int chunks = F / 8;
  const long long n = rows * chunks;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / chunks;
    const int c = static_cast<int>(i - r * chunks);
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + r * 2 * F + c * 8);
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c * 8);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(gh[e]), u = __bfloat1622float2(uh[e]);
      oh[e] = __floats2bfloat162_rn(act_fwd(g.x, act) * u.x, act_fwd(g.y, act) * u.y);
    }
    *reinterpret_cast<uint4*>(out + r * F + c * 8) = o;
  }
}
__global__ void glu_bwd_vec_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                   __nv_bfloat16* __restrict__ dgu, long long rows, int F, int act) {
  const int chunks = F / 8;
  const long long n = rows * chunks;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / chunks;
    const int c = static_cast<int>(i - r * chunks);
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + r * 2 * F + c * 8);
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c * 8);
    const uint4 dv = *reinterpret_cast<const uint4*>(dout + r * F + c * 8);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uv);
    const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&dv);
    uint4 og, ou;
    __nv_bfloat162* ogh = reinterpret_cast<__nv_bfloat162*>(&og);
    __nv_bfloat162* ouh = reinterpret_cast<__nv_bfloat162*>(&ou);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(gh[e]), u = __bfloat1622float2(uh[e]), d = __bfloat1622float2(dh[e]);
      ogh[e] = __floats2bfloat162_rn(d.x * u.x * act_grad(g.x, act), d.y * u.y * act_grad(g.y, act));
      ouh[e] = __floats2bfloat162_rn(d.x * act_fwd(g.x, act), d.y * act_fwd(g.y, act));
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * F + c * 8) = og;
    *reinterpret_cast<uint4*>(dgu + r * 2 * F + F + c * 8) = ou;
  }
}

template <typename T>
__global__ void glu_bwd_kernel(const T* __restrict__ gu, const T* __restrict__ dout, T* __restrict__ dgu,
                               long long rows, int F, int act) {
  long long n = rows * F;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long r = i / F;
    int c = static_cast<int>(i - r * F);
    float g = to_f(gu[r * 2 * F + c]);
    float u = to_f(gu[r * 2 * F + F + c]);
    float d = to_f(dout[i]);
    dgu[r * 2 * F + c] = from_f<T>(d * u * act_grad(g, act));
    dgu[r * 2 * F + F + c] = from_f<T>(d * act_fwd(g, act));
  }
}

template <typename T>
__global__ void embedding_kernel(const long long* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                 long long n_tok, int H, long long vocab, float scale) {
  long long tok = blockIdx.x;
  long long id = ids[tok];
  if (id < 0 || id >= vocab) id = 0;  // never index out of the table
  const T* src = table + id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = to_f(src[i]);
    out[tok * H + i] = from_f<T>(scale == 1.f ? v : v * scale);
  }
}

// W'[o,i] = W[o,i] + sum_r B[o,r] A[r,i]   (A, B fp32; R small)
template <typename T>
__global__ void lora_merge_kernel(const T* __restrict__ w, const float* __restrict__ a, const float* __restrict__ b,
                                  T* __restrict__ out, int O, int I, int R) {
  extern __shared__ float sb[];  // B row for this output row
  int o = blockIdx.x;
  for (int r = threadIdx.x; r < R; r += blockDim.x) sb[r] = b[static_cast<long long>(o) * R + r];
  __syncthreads();
  for (int i = threadIdx.x; i < I; i += blockDim.x) {
    float acc = to_f(w[static_cast<long long>(o) * I + i]);
    for (int r = 0; r < R; ++r) acc += sb[r] * a[static_cast<long long>(r) * I + i];
    out[static_cast<long long>(o) * I + i] = from_f<T>(acc);
  }
}

// ------------------------------------------------------------------ AdamW
// Tensor table lives in device memory: one entry per tensor, chunked over blocks.
__global__ void sumsq_kernel(const AdamTensor* __restrict__ tab, const int* __restrict__ blk_tensor,
                             const long long* __restrict__ blk_off, double* __restrict__ out, int chunk) {
  __shared__ float red[32];
  const AdamTensor t = tab[blk_tensor[blockIdx.x]];
  long long off = blk_off[blockIdx.x];
  long long end = min(off + chunk, t.n);
  float s = 0.f;
  for (long long i = off + threadIdx.x; i < end; i += blockDim.x) {
    float g = t.g[i];
    s += g * g;
  }
  float tot = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, static_cast<double>(tot));
}

// scalars[0] = sum of squares (double, already reduced). clip factor derived on device so no host sync is
// needed between the norm and the update.
__global__ void adamw_kernel(const AdamTensor* __restrict__ tab, const int* __restrict__ blk_tensor,
                             const long long* __restrict__ blk_off, const double* __restrict__ sumsq, int chunk,
                             float lr, float b1, float b2, float eps, float wd, float bc1_inv, float bc2_inv,
                             float max_norm, float pre_scale, float* __restrict__ norm_out) {
  const AdamTensor t = tab[blk_tensor[blockIdx.x]];
  long long off = blk_off[blockIdx.x];
  long long end = min(off + chunk, t.n);
  float gs = pre_scale;
  if (sumsq) {
    float norm = static_cast<float>(sqrt(*sumsq)) * pre_scale;
    if (blockIdx.x == 0 && threadIdx.x == 0 && norm_out) *norm_out = norm;
    if (norm == 0.f) return;  // all-zero gradient: leave parameters and moments untouched
    if (max_norm > 0.f && norm > max_norm) gs *= max_norm / norm;
  }
  for (long long i = off + threadIdx.x; i < end; i += blockDim.x) {
    float g = t.g[i] * gs;
    float m = b1 * t.m[i] + (1.f - b1) * g;
    float v = b2 * t.v[i] + (1.f - b2) * g * g;
    float p = t.p[i] * (1.f - lr * wd);
    p -= lr * (m * bc1_inv) / (sqrtf(v * bc2_inv) + eps);
    t.m[i] = m;
    t.v[i] = v;
    t.p[i] = p;
  }
}

// ------------------------------------------------------------------ GRPO loss
// One block per sequence row. Writes per-row partial sums; the host-side wrapper combines
// them according to the loss type. Also emits dL/dlogp given the upstream scale.
// mode bits: 1 = sequence-level ratio, 2 = has ref, 4 = has tis
__global__ void grpo_loss_kernel(const float* __restrict__ logp, const float* __restrict__ logp_old,
                                 const float* __restrict__ logp_ref, const float* __restrict__ adv,
                                 const float* __restrict__ mask, const float* __restrict__ tis,
                                 float* __restrict__ row_sum, float* __restrict__ row_cnt, float* __restrict__ dlogp,
                                 int L, float eps_lo, float eps_hi, float beta, int mode) {
  __shared__ float red[32];
  const int g = blockIdx.x;
  const float* lp = logp + static_cast<long long>(g) * L;
  const float* lo = logp_old + static_cast<long long>(g) * L;
  const float* lr_ = (mode & 2) ? logp_ref + static_cast<long long>(g) * L : nullptr;
  const float* mk = mask + static_cast<long long>(g) * L;
  const float* tw = (mode & 4) ? tis + static_cast<long long>(g) * L : nullptr;
  const float a = adv[g];
  const float CAP = 60.f;
  float cnt = 0.f, seq_num = 0.f;
  for (int t = threadIdx.x; t < L; t += blockDim.x) {
    float m = mk[t];
    if (m > 0.f) {
      cnt += m;
      seq_num += (lp[t] - lo[t]) * m;
    }
  }
  cnt = block_sum(cnt, red);
  float seq_lr = 0.f;
  bool seq_clamped = false;
  if (mode & 1) {
    seq_num = block_sum(seq_num, red);
    seq_lr = seq_num / fmaxf(cnt, 1.f);
    seq_clamped = (seq_lr < -CAP) || (seq_lr > CAP);
    seq_lr = fminf(fmaxf(seq_lr, -CAP), CAP);
  }
  float acc = 0.f;
  // For the sequence-level ratio every token's surrogate depends on every token's logp through the
  // mean; d(sum_t m_t surr_t)/d logp_u = m_u/cnt * sum_t m_t tis_t dsurr_t/dratio * ratio.
  float seq_coef = 0.f;
  for (int t = threadIdx.x; t < L; t += blockDim.x) {
    float m = mk[t];
    float val = 0.f, dval = 0.f;
    if (m > 0.f) {
      float d = lp[t] - lo[t];
      bool clamped = (mode & 1) ? seq_clamped : (d < -CAP || d > CAP);
      float ratio = __expf((mode & 1) ? seq_lr : fminf(fmaxf(d, -CAP), CAP));
      float un = ratio * a;
      float rc = fminf(fmaxf(ratio, 1.f - eps_lo), 1.f + eps_hi);
      float cl = rc * a;
      float surr = fminf(un, cl);
      // gradient flows through the unclipped branch when it is the minimum (ties go to unclipped)
      float dsurr_dratio = (un <= cl) ? a : ((ratio == rc) ? a : 0.f);
      if (a == 0.f) { surr = 0.f; dsurr_dratio = 0.f; }
      float w = tw ? tw[t] : 1.f;
      surr *= w;
      float dr = clamped ? 0.f : dsurr_dratio * w * ratio;  // d surr / d logp (token level)
      val = surr;
      if (mode & 1) seq_coef += m * dr; else dval = dr;
      if (lr_) {
        float dd = lr_[t] - lp[t];
        float e = __expf(dd);
        val -= beta * (e - dd - 1.f);
        dval += beta * (e - 1.f);  // d(-beta*k3)/dlogp = beta*(e - 1)
      }
      acc += val * m;
    }
    if (dlogp) dlogp[static_cast<long long>(g) * L + t] = dval * m;  // completed below for sequence level
  }
  acc = block_sum(acc, red);
  if (mode & 1) {
    seq_coef = block_sum(seq_coef, red);
    if (dlogp) {
      float per = seq_coef / fmaxf(cnt, 1.f);
      for (int t = threadIdx.x; t < L; t += blockDim.x) {
        float m = mk[t];
        if (m > 0.f) dlogp[static_cast<long long>(g) * L + t] += per * m;
      }
    }
  }
  if (threadIdx.x == 0) {
    row_sum[g] = acc;
    row_cnt[g] = cnt;
  }
}

// dlogp[g,t] *= -(upstream) * row_scale[g]
__global__ void grpo_scale_kernel(float* __restrict__ dlogp, const float* __restrict__ row_scale, long long n, int L) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dlogp[i] *= row_scale[i / L];
}

inline unsigned grid_for(long long n, int threads) {
  long long b = (n + threads - 1) / threads;
  return static_cast<unsigned>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

const char* glu(int dtype, bool backward, const void* gu, const void* dout, void* out, long long rows, int F, int act,
                cudaStream_t s) {
  if (rows * F == 0) return nullptr;
  unsigned grid = grid_for(rows * F, 256);
  if (dtype == kF32) {
    if (backward)
      glu_bwd_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(gu), static_cast<const float*>(dout),
                                                 static_cast<float*>(out), rows, F, act);
    else
      glu_fwd_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(gu), static_cast<float*>(out), rows, F, act);
  } else if ((F % 8) == 0 && (reinterpret_cast<uintptr_t>(gu) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(dout) & 15) == 0) {
    using B = __nv_bfloat16;
    const unsigned vgrid = grid_for(rows * (F / 8), 256);
    if (backward)
      glu_bwd_vec_kernel<<<vgrid, 256, 0, s>>>(static_cast<const B*>(gu), static_cast<const B*>(dout), static_cast<B*>(out),
                                               rows, F, act);
    else
      launch_pdl(glu_fwd_vec_kernel, dim3(vgrid), dim3(256), 0, s, static_cast<const B*>(gu), static_cast<B*>(out), rows, F, act);
  } else {
    using B = __nv_bfloat16;
    if (backward)
      glu_bwd_kernel<B><<<grid, 256, 0, s>>>(static_cast<const B*>(gu), static_cast<const B*>(dout),
                                             static_cast<B*>(out), rows, F, act);
    else
      glu_fwd_kernel<B><<<grid, 256, 0, s>>>(static_cast<const B*>(gu), static_cast<B*>(out), rows, F, act);
  }
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "glu launch failed";
}

const char* embedding(int dtype, const long long* ids, const void* table, void* out, long long n_tok, int H,
                      long long vocab, float scale, cudaStream_t s) {
  if (n_tok == 0) return nullptr;
  if (dtype == kF32)
    embedding_kernel<float><<<static_cast<unsigned>(n_tok), 256, 0, s>>>(ids, static_cast<const float*>(table),
                                                                         static_cast<float*>(out), n_tok, H, vocab, scale);
  else
    embedding_kernel<__nv_bfloat16><<<static_cast<unsigned>(n_tok), 256, 0, s>>>(
        ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), n_tok, H, vocab, scale);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "embedding launch failed";
}

const char* lora_merge(int dtype, const void* w, const float* a, const float* b, void* out, int O, int I, int R,
                       cudaStream_t s) {
  if (O == 0 || I == 0) return nullptr;
  size_t sm = static_cast<size_t>(R) * sizeof(float);
  if (dtype == kF32)
    lora_merge_kernel<float><<<O, 256, sm, s>>>(static_cast<const float*>(w), a, b, static_cast<float*>(out), O, I, R);
  else
    lora_merge_kernel<__nv_bfloat16><<<O, 256, sm, s>>>(static_cast<const __nv_bfloat16*>(w), a, b,
                                                        static_cast<__nv_bfloat16*>(out), O, I, R);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "lora_merge launch failed";
}

const char* adamw_multi(const AdamTensor* tab_dev, const int* blk_tensor_dev, const long long* blk_off_dev,
                        int n_blocks, int chunk, double* sumsq_dev, bool compute_norm, float lr, float b1, float b2,
                        float eps, float wd, float bc1_inv, float bc2_inv, float max_norm, float pre_scale,
                        float* norm_out_dev, cudaStream_t s) {
  if (n_blocks == 0) return nullptr;
  if (compute_norm) {
    cudaMemsetAsync(sumsq_dev, 0, sizeof(double), s);
    sumsq_kernel<<<n_blocks, 256, 0, s>>>(tab_dev, blk_tensor_dev, blk_off_dev, sumsq_dev, chunk);
    count_launch();
  }
  adamw_kernel<<<n_blocks, 256, 0, s>>>(tab_dev, blk_tensor_dev, blk_off_dev, compute_norm ? sumsq_dev : nullptr, chunk, lr, b1, b2, eps, wd,
                                        bc1_inv, bc2_inv, max_norm, pre_scale, norm_out_dev);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "adamw launch failed";
}

const char* grpo_loss_rows(const float* logp, const float* logp_old, const float* logp_ref, const float* adv,
                           const float* mask, const float* tis, float* row_sum, float* row_cnt, float* dlogp, int G,
                           int L, float eps_lo, float eps_hi, float beta, int mode, cudaStream_t s) {
  if (G == 0) return nullptr;
  grpo_loss_kernel<<<G, 256, 0, s>>>(logp, logp_old, logp_ref, adv, mask, tis, row_sum, row_cnt, dlogp, L, eps_lo,
                                     eps_hi, beta, mode);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "grpo_loss launch failed";
}

const char* grpo_scale_rows(float* dlogp, const float* row_scale, int G, int L, cudaStream_t s) {
  long long n = static_cast<long long>(G) * L;
  if (n == 0) return nullptr;
  grpo_scale_kernel<<<grid_for(n, 256), 256, 0, s>>>(dlogp, row_scale, n, L);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "grpo_scale launch failed";
}

}  // namespace ferrl
