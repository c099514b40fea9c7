// RMSNorm family and RoPE for sm_100a: bandwidth-bound row kernels.
//
//   rmsnorm            y = x * rsqrt(mean(x^2)+eps) * w        (w or 1+w)
//   add_rmsnorm        h = x + res (written back), y = rmsnorm(h)
//   rmsnorm_gated      y = rmsnorm(x) * w * silu(gate)
//   rmsnorm_bwd        dx for a frozen weight (LoRA training never needs dw)
//   qk_norm_rope       per-head RMSNorm of q and k fused with rotate-half RoPE (full or
//                      partial rotary width), reading the fused qkv GEMM output in place
//                      and writing contiguous q / k; optional direct write of k, v into a
//                      KV cache row at each sequence's current length (decode)
//   qk_norm_rope_bwd   inverse rotation + norm backward
//
// One row per CTA (hidden-size rows) or one head-row per warp (head_dim rows); 16-byte
// vector loads; fp32 math; each element is read once and written once.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"

namespace ferrl {
namespace {

template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w,
                               const T* __restrict__ gate, T* __restrict__ y, T* __restrict__ h_out, int H, float eps,
                               int zero_centered) {
  pdl_trigger();   // a dependent GEMM may start streaming its weights while this kernel runs
  pdl_wait();      // launched as a programmatic dependent itself: nothing is read before the predecessor is done
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * H;
  const T* rr = res ? res + row * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = to_f(xr[i]);
    if (rr) {
      v += to_f(rr[i]);
      // round through the storage type so the norm sees exactly what the residual stream holds
      T hv = from_f<T>(v);
      h_out[row * H + i] = hv;
      v = to_f(hv);
    }
    ss += v * v;
  }
  float tot = block_sum(ss, red);
  float rstd = rsqrtf(tot / H + eps);
  const T* src = rr ? h_out + row * H : xr;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = to_f(src[i]) * rstd;
    if (w) {
      float wv = to_f(w[i]);
      v *= zero_centered ? (1.f + wv) : wv;
    }
    if (gate) {
      float g = to_f(gate[row * H + i]);
      v *= g / (1.f + __expf(-g));
    }
    y[row * H + i] = from_f<T>(v);
  }
}

// dx_i = rstd * (w_i dy_i - x_i * rstd^2 * mean_j(w_j dy_j x_j))
template <typename T>
__global__ void rmsnorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ dy,
                                   T* __restrict__ dx, int H, float eps, int zero_centered) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * H;
  const T* gr = dy + row * H;
  float ss = 0.f, dot = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = to_f(xr[i]);
    float wv = w ? to_f(w[i]) : 1.f;
    if (zero_centered) wv += 1.f;
    ss += v * v;
    dot += v * wv * to_f(gr[i]);
  }
  float tot = block_sum(ss, red);
  float d = block_sum(dot, red);
  float rstd = rsqrtf(tot / H + eps);
  float c = d * rstd * rstd / H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = to_f(xr[i]);
    float wv = w ? to_f(w[i]) : 1.f;
    if (zero_centered) wv += 1.f;
    dx[row * H + i] = from_f<T>(rstd * (wv * to_f(gr[i]) - v * c));
  }
}

// ---- bf16 vector forms: each thread owns up to VMAX 16-byte chunks of the row and keeps them in
// registers between the reduction and the scaling, so every byte is read once and all accesses
// are 16 bytes wide.  Same arithmetic (and the same rounding points) as the scalar kernels above.
constexpr int VMAX = 4;

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float2 t = __bfloat1622float2(h[e]);
    f[2 * e] = t.x;
    f[2 * e + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8f(const float* f) {
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
  return o;
}

__global__ void rmsnorm_vec_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ gate,
                                   __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out, int H, float eps,
                                   int zero_centered) {
  pdl_trigger();   // a dependent GEMM may start streaming its weights while this kernel runs
  pdl_wait();      // launched as a programmatic dependent itself: nothing is read before the predecessor is done
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int chunks = H / 8;
  float v[VMAX][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VMAX; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      unpack8(reinterpret_cast<const uint4*>(x + row * H)[c], v[k]);
      if (res) {
        float r[8];
        unpack8(reinterpret_cast<const uint4*>(res + row * H)[c], r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[k][e] += r[e];
        const uint4 hv = pack8f(v[k]);          // the norm sees exactly what the residual stream holds
        reinterpret_cast<uint4*>(h_out + row * H)[c] = hv;
        unpack8(hv, v[k]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[k][e] * v[k][e];
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / H + eps);
#pragma unroll
  for (int k = 0; k < VMAX; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[k][e] * rstd;
      if (w) {
        float wv[8];
        unpack8(reinterpret_cast<const uint4*>(w)[c], wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] *= zero_centered ? (1.f + wv[e]) : wv[e];
      }
      if (gate) {
        float g[8];
        unpack8(reinterpret_cast<const uint4*>(gate + row * H)[c], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] *= g[e] / (1.f + __expf(-g[e]));
      }
      reinterpret_cast<uint4*>(y + row * H)[c] = pack8f(o);
    }
  }
}

__global__ void rmsnorm_bwd_vec_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                       const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, int H,
                                       float eps, int zero_centered) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int chunks = H / 8;
  float xv[VMAX][8], gw[VMAX][8];      // x and w*dy
  float ss = 0.f, dot = 0.f;
#pragma unroll
  for (int k = 0; k < VMAX; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      unpack8(reinterpret_cast<const uint4*>(x + row * H)[c], xv[k]);
      unpack8(reinterpret_cast<const uint4*>(dy + row * H)[c], gw[k]);
      float wv[8];
      if (w) unpack8(reinterpret_cast<const uint4*>(w)[c], wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float ww = w ? wv[e] : 1.f;
        if (zero_centered) ww += 1.f;
        gw[k][e] *= ww;
        ss += xv[k][e] * xv[k][e];
        dot += xv[k][e] * gw[k][e];
      }
    }
  }
  const float tot = block_sum(ss, red);
  const float d = block_sum(dot, red);
  const float rstd = rsqrtf(tot / H + eps);
  const float cc = d * rstd * rstd / H;
#pragma unroll
  for (int k = 0; k < VMAX; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < chunks) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = rstd * (gw[k][e] - xv[k][e] * cc);
      reinterpret_cast<uint4*>(dx + row * H)[c] = pack8f(o);
    }
  }
}

static inline bool vec_ok(int H, const void* a, const void* b, const void* c, const void* d, const void* e, const void* f) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return (H % 8) == 0 && H / 8 <= VMAX * 512 && al(a) && al(b) && al(c) && al(d) && al(e) && al(f);
}
static inline int vec_threads(int H) {
  const int chunks = H / 8;
  int t = (chunks + VMAX - 1) / VMAX;
  t = (t + 31) / 32 * 32;
  return t < 64 ? 64 : (t > 512 ? 512 : t);
}

// One warp per (token, head). D <= 512, D even. rot = 2*half <= D.
template <typename T, bool BWD>
__global__ void qk_norm_rope_kernel(const T* __restrict__ q_in, long long ld_q, const T* __restrict__ k_in,
                                    long long ld_k, long long ld_dq, long long ld_dk, const T* __restrict__ qw, const T* __restrict__ kw,
                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                    const long long* __restrict__ pos, const int* __restrict__ pos32, int pos_div,
                                    T* __restrict__ q_out, T* __restrict__ k_out, const T* __restrict__ dq,
                                    const T* __restrict__ dk, long long n_tok, int Hq, int Hkv, int D, int half,
                                    float eps, int zero_centered) {
  const int warps_per_block = blockDim.x >> 5;
  const long long wid = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = Hq + Hkv;
  if (wid >= n_tok * heads) return;
  const long long tok = wid / heads;
  const int hh = static_cast<int>(wid % heads);
  const bool is_q = hh < Hq;
  const int h = is_q ? hh : hh - Hq;
  const T* src = (is_q ? q_in + tok * ld_q : k_in + tok * ld_k) + h * D;
  const T* wv = is_q ? qw : kw;
  const long long p = pos ? pos[tok / pos_div] : static_cast<long long>(pos32[tok / pos_div]);
  const float* cr = cos_t + p * half;
  const float* sr = sin_t + p * half;
  const int rot = 2 * half;
  constexpr int MAXE = 16;  // D <= 512
  float xv[MAXE];
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < MAXE; ++e) {
    int i = lane + 32 * e;
    xv[e] = (i < D) ? to_f(src[i]) : 0.f;
    ss += xv[e] * xv[e];
  }
  float rstd = 1.f;
  if (wv) {
    ss = warp_sum(ss);
    rstd = rsqrtf(ss / D + eps);
  }
  if (!BWD) {
    T* dst = (is_q ? q_out + (tok * Hq + h) * D : k_out + (tok * Hkv + h) * D);
    // normalise, then rotate pairs (i, i+half). The partner value comes from a shuffle-free
    // re-read of registers: element i lives in lane i%32 slot i/32; its partner i+half has the
    // same lane when half % 32 == 0, otherwise fall back to shared-free global re-read.
#pragma unroll
    for (int e = 0; e < MAXE; ++e) {
      int i = lane + 32 * e;
      if (i >= D) break;
      float w0 = wv ? to_f(wv[i]) + (zero_centered ? 1.f : 0.f) : 1.f;
      float v = xv[e] * rstd * w0;
      if (i < rot) {
        int j = (i < half) ? i + half : i - half;
        float wj = wv ? to_f(wv[j]) + (zero_centered ? 1.f : 0.f) : 1.f;
        float u = to_f(src[j]) * rstd * wj;
        // round the normalised values through T as the unfused reference does
        v = to_f(from_f<T>(v));
        u = to_f(from_f<T>(u));
        int f = (i < half) ? i : i - half;
        float c = cr[f], s = sr[f];
        v = (i < half) ? (v * c - u * s) : (v * c + u * s);
      }
      dst[i] = from_f<T>(v);
    }
  } else {
    // g = d(out); first undo the rotation: dn_i = g_i c + g_{i+half} s (i<half); dn_i = g_i c - g_{i-half} s
    const T* g = is_q ? dq + (tok * Hq + h) * D : dk + (tok * Hkv + h) * D;
    float dn[MAXE];
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < MAXE; ++e) {
      int i = lane + 32 * e;
      dn[e] = 0.f;
      if (i < D) {
        float gi = to_f(g[i]);
        if (i < rot) {
          int j = (i < half) ? i + half : i - half;
          int f = (i < half) ? i : i - half;
          float gj = to_f(g[j]);
          float c = cr[f], s = sr[f];
          gi = (i < half) ? (gi * c + gj * s) : (gi * c - gj * s);
        }
        dn[e] = gi;
        float w0 = wv ? to_f(wv[i]) + (zero_centered ? 1.f : 0.f) : 1.f;
        dot += xv[e] * w0 * gi;
      }
    }
    // in backward q_out / k_out are the destinations of d(q_in) / d(k_in) with their own token strides
    T* dst = (is_q ? q_out + tok * ld_dq : k_out + tok * ld_dk) + h * D;
    if (wv) {
      dot = warp_sum(dot);
      float c2 = dot * rstd * rstd / D;
#pragma unroll
      for (int e = 0; e < MAXE; ++e) {
        int i = lane + 32 * e;
        if (i >= D) break;
        float w0 = to_f(wv[i]) + (zero_centered ? 1.f : 0.f);
        dst[i] = from_f<T>(rstd * (w0 * dn[e] - xv[e] * c2));
      }
    } else {
#pragma unroll
      for (int e = 0; e < MAXE; ++e) {
        int i = lane + 32 * e;
        if (i >= D) break;
        dst[i] = from_f<T>(dn[e]);
      }
    }
  }
}

// bf16 vector form for D = 32*EPL (128 or 256): one warp per (token, head), EPL consecutive
// channels per lane in one 8- or 16-byte access, rotation partners fetched with a warp shuffle
// (partner lane = lane +- half/EPL).  Same arithmetic and rounding points as the kernel above.
template <int EPL, bool BWD>
__global__ void qk_norm_rope_vec_kernel(const __nv_bfloat16* __restrict__ q_in, long long ld_q,
                                        const __nv_bfloat16* __restrict__ k_in, long long ld_k, long long ld_dq,
                                        long long ld_dk, const __nv_bfloat16* __restrict__ qw,
                                        const __nv_bfloat16* __restrict__ kw, const float* __restrict__ cos_t,
                                        const float* __restrict__ sin_t, const long long* __restrict__ pos,
                                        const int* __restrict__ pos32, int pos_div, __nv_bfloat16* __restrict__ q_out,
                                        __nv_bfloat16* __restrict__ k_out, const __nv_bfloat16* __restrict__ dq,
                                        const __nv_bfloat16* __restrict__ dk, long long n_tok, int Hq, int Hkv, int half,
                                        float eps, int zero_centered, __nv_bfloat16* __restrict__ kc,
                                        __nv_bfloat16* __restrict__ vc, const __nv_bfloat16* __restrict__ v_in, long long ld_v,
                                        const int* __restrict__ kv_len, const int* __restrict__ table, int bt_stride, int page,
                                        int smax) {
  pdl_trigger();
  pdl_wait();      // may be launched as a programmatic dependent: nothing is read before the predecessor is done
  constexpr int D = 32 * EPL;
  const long long wid = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = Hq + Hkv;
  if (wid >= n_tok * heads) return;          // warp-uniform
  const long long tok = wid / heads;
  const int hh = static_cast<int>(wid % heads);
  const bool is_q = hh < Hq;
  const int h = is_q ? hh : hh - Hq;
  const __nv_bfloat16* src = (is_q ? q_in + tok * ld_q : k_in + tok * ld_k) + h * D + lane * EPL;
  const __nv_bfloat16* wv = is_q ? qw : kw;
  const long long p = pos ? pos[tok / pos_div] : static_cast<long long>(pos32[tok / pos_div]);
  const int rot = 2 * half;
  const int i0 = lane * EPL;
  const int shift = half / EPL;                                  // lanes between rotation partners
  const bool in_rot = i0 < rot, lower = i0 < half;
  const int partner = in_rot ? (lower ? lane + shift : lane - shift) : lane;

  auto load = [&](const __nv_bfloat16* ptr, float* f) {
    if (EPL == 4) {
      const uint2 v = *reinterpret_cast<const uint2*>(ptr);
      const __nv_bfloat162* hh2 = reinterpret_cast<const __nv_bfloat162*>(&v);
      float2 a = __bfloat1622float2(hh2[0]), b = __bfloat1622float2(hh2[1]);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
    } else {
      unpack8(*reinterpret_cast<const uint4*>(ptr), f);
    }
  };
  auto store = [&](__nv_bfloat16* ptr, const float* f) {
    if (EPL == 4) {
      uint2 v;
      __nv_bfloat162* hh2 = reinterpret_cast<__nv_bfloat162*>(&v);
      hh2[0] = __floats2bfloat162_rn(f[0], f[1]);
      hh2[1] = __floats2bfloat162_rn(f[2], f[3]);
      *reinterpret_cast<uint2*>(ptr) = v;
    } else {
      *reinterpret_cast<uint4*>(ptr) = pack8f(f);
    }
  };

  float x[EPL], w[EPL], c[EPL], sn[EPL];
  load(src, x);
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    ss += x[e] * x[e];
    w[e] = 1.f;
    c[e] = 1.f;
    sn[e] = 0.f;
  }
  float rstd = 1.f;
  if (wv) {
    load(wv + i0, w);
    if (zero_centered) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) w[e] += 1.f;
    }
    rstd = rsqrtf(warp_sum(ss) / D + eps);
  }
  if (in_rot) {
    const int f0 = lower ? i0 : i0 - half;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      c[e] = cos_t[p * half + f0 + e];
      sn[e] = sin_t[p * half + f0 + e];
    }
  }
  if (!BWD) {
    float v[EPL], o[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      v[e] = x[e] * rstd * w[e];
      // the unfused form rounds the normalised value to bf16 before rotating it
      if (in_rot) v[e] = __bfloat162float(__float2bfloat16_rn(v[e]));
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float u = __shfl_sync(0xffffffffu, v[e], partner);
      o[e] = in_rot ? (lower ? v[e] * c[e] - u * sn[e] : v[e] * c[e] + u * sn[e]) : v[e];
    }
    if (!is_q && kc) {
      // decode: the key goes to its cache row, and the value row of the same head is copied along
      const int t = kv_len[tok];
      const long long slot = table ? static_cast<long long>(table[tok * bt_stride + t / page]) * page + t % page
                                   : tok * smax + t;
      const long long off = (slot * Hkv + h) * D + i0;
      store(kc + off, o);
      float vv[EPL];
      load(v_in + tok * ld_v + h * D + i0, vv);
      store(vc + off, vv);
    } else {
      store((is_q ? q_out + (tok * Hq + h) * D : k_out + (tok * Hkv + h) * D) + i0, o);
    }
  } else {
    float g[EPL], dn[EPL];
    load((is_q ? dq + (tok * Hq + h) * D : dk + (tok * Hkv + h) * D) + i0, g);
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float gj = __shfl_sync(0xffffffffu, g[e], partner);
      dn[e] = in_rot ? (lower ? g[e] * c[e] + gj * sn[e] : g[e] * c[e] - gj * sn[e]) : g[e];
      dot += x[e] * w[e] * dn[e];
    }
    __nv_bfloat16* dst = (is_q ? q_out + tok * ld_dq : k_out + tok * ld_dk) + h * D + i0;
    float o[EPL];
    if (wv) {
      const float c2 = warp_sum(dot) * rstd * rstd / D;
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[e] = rstd * (w[e] * dn[e] - x[e] * c2);
    } else {
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[e] = dn[e];
    }
    store(dst, o);
  }
}

// Decode: append this step's k (already normed+roped, [B,Hkv,D]) and v (view into qkv) to the cache
// at each row's current length.
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k, const T* __restrict__ v, long long ldv, T* __restrict__ kc,
                                 T* __restrict__ vc, const int* __restrict__ kv_len, int smax, int HD) {
  pdl_trigger();
  pdl_wait();      // may be launched as a programmatic dependent: nothing is read before the predecessor is done
  const int b = blockIdx.x;
  const long long slot = static_cast<long long>(b) * smax + kv_len[b];
  if (kv_len[b] >= smax) return;  // cache full: drop rather than write out of bounds
  for (int i = threadIdx.x; i < HD; i += blockDim.x) {
    kc[slot * HD + i] = k[static_cast<long long>(b) * HD + i];
    vc[slot * HD + i] = v[static_cast<long long>(b) * ldv + i];
  }
}

}  // namespace

template <typename T>
static const char* rmsnorm_t(const void* x, const void* res, const void* w, const void* gate, void* y, void* h_out,
                             long long rows, int H, float eps, bool zc, cudaStream_t s) {
  if (rows == 0) return nullptr;
  if (sizeof(T) == 2 && vec_ok(H, x, res, w, gate, y, h_out)) {
    using B = __nv_bfloat16;
    launch_pdl(rmsnorm_vec_kernel, dim3(static_cast<unsigned>(rows)), dim3(vec_threads(H)), 0, s,
               static_cast<const B*>(x), static_cast<const B*>(res), static_cast<const B*>(w), static_cast<const B*>(gate),
               static_cast<B*>(y), static_cast<B*>(h_out), H, eps, zc ? 1 : 0);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? nullptr : "rmsnorm launch failed";
  }
  int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  rmsnorm_kernel<T><<<static_cast<unsigned>(rows), threads, 0, s>>>(
      static_cast<const T*>(x), static_cast<const T*>(res), static_cast<const T*>(w), static_cast<const T*>(gate),
      static_cast<T*>(y), static_cast<T*>(h_out), H, eps, zc ? 1 : 0);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "rmsnorm launch failed";
}

const char* rmsnorm(int dtype, const void* x, const void* res, const void* w, const void* gate, void* y, void* h_out,
                    long long rows, int H, float eps, bool zero_centered, cudaStream_t s) {
  return dtype == kF32 ? rmsnorm_t<float>(x, res, w, gate, y, h_out, rows, H, eps, zero_centered, s)
                       : rmsnorm_t<__nv_bfloat16>(x, res, w, gate, y, h_out, rows, H, eps, zero_centered, s);
}

template <typename T>
static const char* rmsnorm_bwd_t(const void* x, const void* w, const void* dy, void* dx, long long rows, int H,
                                 float eps, bool zc, cudaStream_t s) {
  if (rows == 0) return nullptr;
  if (sizeof(T) == 2 && vec_ok(H, x, w, dy, dx, nullptr, nullptr)) {
    using B = __nv_bfloat16;
    rmsnorm_bwd_vec_kernel<<<static_cast<unsigned>(rows), vec_threads(H), 0, s>>>(
        static_cast<const B*>(x), static_cast<const B*>(w), static_cast<const B*>(dy), static_cast<B*>(dx), H, eps,
        zc ? 1 : 0);
    count_launch();
    return cudaGetLastError() == cudaSuccess ? nullptr : "rmsnorm_bwd launch failed";
  }
  int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  rmsnorm_bwd_kernel<T><<<static_cast<unsigned>(rows), threads, 0, s>>>(
      static_cast<const T*>(x), static_cast<const T*>(w), static_cast<const T*>(dy), static_cast<T*>(dx), H, eps,
      zc ? 1 : 0);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "rmsnorm_bwd launch failed";
}

const char* rmsnorm_bwd(int dtype, const void* x, const void* w, const void* dy, void* dx, long long rows, int H,
                        float eps, bool zero_centered, cudaStream_t s) {
  return dtype == kF32 ? rmsnorm_bwd_t<float>(x, w, dy, dx, rows, H, eps, zero_centered, s)
                       : rmsnorm_bwd_t<__nv_bfloat16>(x, w, dy, dx, rows, H, eps, zero_centered, s);
}

// Gated RMSNorm backward with a frozen weight: y = x * rstd * w * silu(g).
//   a_i = dy_i w_i silu(g_i);  dx_i = rstd (a_i - x_i rstd^2 mean_j(a_j x_j));  dg_i = dy_i x_i rstd w_i silu'(g_i)
// One warp per row (rows are GatedDeltaNet value heads, H = 128), several rows per CTA.
template <typename T>
__global__ void rmsnorm_gated_bwd_kernel(const T* __restrict__ x, const T* __restrict__ gate, const T* __restrict__ w,
                                         const T* __restrict__ dy, T* __restrict__ dx, T* __restrict__ dg, long long rows,
                                         int H, float eps) {
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const T* xr = x + row * H;
  const T* gr = gate + row * H;
  const T* yr = dy + row * H;
  float ss = 0.f, dot = 0.f;
  for (int i = lane; i < H; i += 32) {
    const float v = to_f(xr[i]), g = to_f(gr[i]);
    const float sg = 1.f / (1.f + __expf(-g));
    ss += v * v;
    dot += v * to_f(yr[i]) * to_f(w[i]) * g * sg;
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float rstd = rsqrtf(ss / H + eps);
  const float c = dot * rstd * rstd / H;
  for (int i = lane; i < H; i += 32) {
    const float v = to_f(xr[i]), g = to_f(gr[i]), d = to_f(yr[i]) * to_f(w[i]);
    const float sg = 1.f / (1.f + __expf(-g));
    dx[row * H + i] = from_f<T>(rstd * (d * g * sg - v * c));
    dg[row * H + i] = from_f<T>(d * v * rstd * sg * (1.f + g * (1.f - sg)));
  }
}

template <typename T>
static const char* rmsnorm_gated_bwd_t(const void* x, const void* gate, const void* w, const void* dy, void* dx, void* dg,
                                       long long rows, int H, float eps, cudaStream_t s) {
  if (rows == 0) return nullptr;
  const int warps = 8;
  rmsnorm_gated_bwd_kernel<T><<<static_cast<unsigned>((rows + warps - 1) / warps), warps * 32, 0, s>>>(
      static_cast<const T*>(x), static_cast<const T*>(gate), static_cast<const T*>(w), static_cast<const T*>(dy),
      static_cast<T*>(dx), static_cast<T*>(dg), rows, H, eps);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "rmsnorm_gated_bwd launch failed";
}

const char* rmsnorm_gated_bwd(int dtype, const void* x, const void* gate, const void* w, const void* dy, void* dx,
                              void* dg, long long rows, int H, float eps, cudaStream_t s) {
  return dtype == kF32 ? rmsnorm_gated_bwd_t<float>(x, gate, w, dy, dx, dg, rows, H, eps, s)
                       : rmsnorm_gated_bwd_t<__nv_bfloat16>(x, gate, w, dy, dx, dg, rows, H, eps, s);
}

template <typename T, bool BWD>
static const char* qknr_t(const QkNormRopeArgs& a, cudaStream_t s) {
  if (a.D > 512 || (a.D & 1) || 2 * a.half > a.D) return "qk_norm_rope: head_dim must be even, <= 512, rot <= D";
  long long units = a.n_tok * (a.Hq + a.Hkv);
  if (units == 0) return nullptr;
  int wpb = 8;
  long long blocks = (units + wpb - 1) / wpb;
  if (sizeof(T) == 2 && (a.D == 128 || a.D == 256)) {
    const int epl = a.D / 32;
    auto al = [&](const void* p, long long ld) { return (reinterpret_cast<uintptr_t>(p) % (2 * epl)) == 0 && (ld % epl) == 0; };
    const bool ok = (a.half % epl) == 0 && al(a.q_in, a.ld_q) && al(a.k_in, a.ld_k) && al(a.q_out, a.backward ? a.ld_dq : epl) &&
                    al(a.k_out, a.backward ? a.ld_dk : epl) && al(a.qw, epl) && al(a.kw, epl) && al(a.dq, epl) && al(a.dk, epl) &&
                    (!a.kc || (!BWD && al(a.kc, epl) && al(a.vc, epl) && al(a.v_in, a.ld_v) && a.kv_len));
    if (ok) {
      using B = __nv_bfloat16;
#define FERRL_QKV(EPLV)                                                                                             \
  launch_pdl(qk_norm_rope_vec_kernel<EPLV, BWD>, dim3(static_cast<unsigned>(blocks)), dim3(wpb * 32), 0, s,          \
      static_cast<const B*>(a.q_in), a.ld_q, static_cast<const B*>(a.k_in), a.ld_k, a.ld_dq, a.ld_dk,               \
      static_cast<const B*>(a.qw), static_cast<const B*>(a.kw), a.cos_t, a.sin_t, a.pos64, a.pos32, a.pos_div,      \
      static_cast<B*>(a.q_out), static_cast<B*>(a.k_out), static_cast<const B*>(a.dq), static_cast<const B*>(a.dk), \
      a.n_tok, a.Hq, a.Hkv, a.half, a.eps, a.zero_centered ? 1 : 0, static_cast<B*>(a.kc), static_cast<B*>(a.vc),      \
      static_cast<const B*>(a.v_in), a.ld_v, a.kv_len, a.table, a.bt_stride, a.page, a.smax)
      if (epl == 4) FERRL_QKV(4); else FERRL_QKV(8);
#undef FERRL_QKV
      count_launch();
      return cudaGetLastError() == cudaSuccess ? nullptr : "qk_norm_rope launch failed";
    }
  }
  if (a.kc) return "qk_norm_rope: the fused cache append needs bf16 heads of 128 or 256 and aligned rows";
  qk_norm_rope_kernel<T, BWD><<<static_cast<unsigned>(blocks), wpb * 32, 0, s>>>(
      static_cast<const T*>(a.q_in), a.ld_q, static_cast<const T*>(a.k_in), a.ld_k, a.ld_dq, a.ld_dk,
      static_cast<const T*>(a.qw),
      static_cast<const T*>(a.kw), a.cos_t, a.sin_t, a.pos64, a.pos32, a.pos_div, static_cast<T*>(a.q_out),
      static_cast<T*>(a.k_out), static_cast<const T*>(a.dq), static_cast<const T*>(a.dk), a.n_tok, a.Hq, a.Hkv, a.D,
      a.half, a.eps, a.zero_centered ? 1 : 0);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "qk_norm_rope launch failed";
}

const char* qk_norm_rope(const QkNormRopeArgs& a, cudaStream_t s) {
  if (a.dtype == kF32) return a.backward ? qknr_t<float, true>(a, s) : qknr_t<float, false>(a, s);
  return a.backward ? qknr_t<__nv_bfloat16, true>(a, s) : qknr_t<__nv_bfloat16, false>(a, s);
}

namespace {
// Paged form: the caches are a pool [n_pages, page, Hkv*D]; row b's token t lives in page
// table[b, t / page] at offset t % page.
__global__ void kv_append_paged_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, long long ldv,
                                       __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc,
                                       const int* __restrict__ kv_len, const int* __restrict__ table, int bt_stride,
                                       int page, int HD) {
  pdl_trigger();
  pdl_wait();      // may be launched as a programmatic dependent: nothing is read before the predecessor is done
  const int b = blockIdx.x;
  const int t = kv_len[b];
  if (t / page >= bt_stride) return;   // row is full: drop rather than write out of bounds
  const long long slot = static_cast<long long>(table[static_cast<long long>(b) * bt_stride + t / page]) * page + t % page;
  for (int i = threadIdx.x; i < HD / 8; i += blockDim.x) {
    reinterpret_cast<uint4*>(kc + slot * HD)[i] = reinterpret_cast<const uint4*>(k + static_cast<long long>(b) * HD)[i];
    reinterpret_cast<uint4*>(vc + slot * HD)[i] = reinterpret_cast<const uint4*>(v + static_cast<long long>(b) * ldv)[i];
  }
}
}  // namespace

// ss[row] = sum of squares of a bf16 row (one warp per row): the first link of the chain of folded
// RMSNorms in the decode loop, whose later links come out of the projections' epilogues.
__global__ void row_sumsq_kernel(const __nv_bfloat16* __restrict__ x, long long ld, float* __restrict__ ss, int rows, int H) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * ld;
  float acc = 0.f;
  for (int i = lane * 8; i < H; i += 256) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      acc += f.x * f.x + f.y * f.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) ss[row] = acc;
}

const char* row_sumsq(const void* x, long long ld, float* ss, int rows, int H, cudaStream_t s) {
  if (rows == 0) return nullptr;
  if ((H % 8) || (ld % 8) || (reinterpret_cast<uintptr_t>(x) & 15)) return "row_sumsq: bf16 rows of a multiple of 8, 16-byte aligned";
  launch_pdl(row_sumsq_kernel, dim3((rows + 7) / 8), dim3(256), 0, s, static_cast<const __nv_bfloat16*>(x), ld, ss, rows, H);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "row_sumsq launch failed";
}

const char* kv_append_paged(const void* k, const void* v, long long ldv, void* kc, void* vc, const int* kv_len,
                            const int* table, int bt_stride, int page, int batch, int HD, cudaStream_t s) {
  if (batch == 0) return nullptr;
  if ((HD % 8) || (ldv % 8) || (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (reinterpret_cast<uintptr_t>(kc) & 15) || (reinterpret_cast<uintptr_t>(vc) & 15))
    return "kv_append_paged: 16-byte aligned rows required";
  launch_pdl(kv_append_paged_kernel, dim3(batch), dim3(128), 0, s, static_cast<const __nv_bfloat16*>(k),
             static_cast<const __nv_bfloat16*>(v), ldv, static_cast<__nv_bfloat16*>(kc), static_cast<__nv_bfloat16*>(vc), kv_len, table,
             bt_stride, page, HD);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "kv_append_paged launch failed";
}

const char* kv_append(int dtype, const void* k, const void* v, long long ldv, void* kc, void* vc, const int* kv_len,
                      int batch, int smax, int HD, cudaStream_t s) {
  if (batch == 0) return nullptr;
  if (dtype == kF32)
    kv_append_kernel<float><<<batch, 256, 0, s>>>(static_cast<const float*>(k), static_cast<const float*>(v), ldv,
                                                  static_cast<float*>(kc), static_cast<float*>(vc), kv_len, smax, HD);
  else
    launch_pdl(kv_append_kernel<__nv_bfloat16>, dim3(batch), dim3(256), 0, s,
               static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), ldv,
               static_cast<__nv_bfloat16*>(kc), static_cast<__nv_bfloat16*>(vc), kv_len, smax, HD);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "kv_append launch failed";
}

}  // namespace ferrl
