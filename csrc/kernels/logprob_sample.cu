// Vocabulary-wide row kernels for sm_100a.
//
//   logprob_rows      per row: log_softmax(f(logit)/T)[target] with an online (single read) max/sum;
//                     f = identity or cap*tanh(x/cap); keeps the row's log-sum-exp for backward
//   logprob_rows_bwd  overwrites the logits row in place with d(loss)/d(logit)
//                     = dlp * (onehot - softmax) * f'(x) / T, ready to feed the dX GEMM
//   sample_rows       temperature + nucleus (top-p) sampling, one CTA per row, counter RNG keyed by
//                     (seed, global row, draw); returns token and behaviour log-prob
//
// sample_rows does all probability mass arithmetic in 2^-40 fixed point with integer atomics, so
// the nucleus threshold and the drawn token do not depend on the order in which threads add
// (bit-reproducible across runs).  The nucleus threshold is found with a 4-pass radix select over
// the float bit pattern of the unnormalised probabilities - no sort, no host copy of the row.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"

namespace ferrl {
namespace {

__device__ __forceinline__ float capf(float x, float cap) { return cap > 0.f ? cap * tanhf(x / cap) : x; }

template <typename T>
__global__ void logprob_rows_kernel(const T* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                                    float* __restrict__ lp, float* __restrict__ lse, int V, float inv_t, float cap) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float z = capf(to_f(x[i]), cap) * inv_t;
    if (z > m) {
      s = s * __expf(m - z) + 1.f;
      m = z;
    } else {
      s += __expf(z - m);
    }
  }
  float gm = block_max(m, red);
  float part = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  float tot = block_sum(part, red);
  if (threadIdx.x == 0) {
    float l = gm + logf(tot);
    long long t = targets[row];
    float zt = (t >= 0 && t < V) ? capf(to_f(x[t]), cap) * inv_t : -INFINITY;
    lp[row] = zt - l;
    lse[row] = l;
  }
}

template <typename T>
__global__ void logprob_rows_bwd_kernel(T* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                                        const float* __restrict__ lse, const float* __restrict__ dlp, int V,
                                        float inv_t, float cap) {
  const long long row = blockIdx.x;
  T* x = logits + row * ld;
  const float l = lse[row], g = dlp[row];
  const long long t = targets[row];
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float raw = to_f(x[i]);
    float y = capf(raw, cap);
    float p = __expf(y * inv_t - l);
    float d = g * ((i == t ? 1.f : 0.f) - p) * inv_t;
    if (cap > 0.f) {
      float th = y / cap;
      d *= (1.f - th * th);
    }
    x[i] = from_f<T>(d);
  }
}

// bf16 vector forms: 8 logits per 16-byte access, so a thread keeps eight times the bytes in flight
// (the scalar kernels above run at a fifth of the copy bandwidth because they are latency-bound).
__global__ void logprob_rows_vec_kernel(const __nv_bfloat16* __restrict__ logits, long long ld,
                                        const long long* __restrict__ targets, float* __restrict__ lp,
                                        float* __restrict__ lse, int V, float inv_t, float cap) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* x = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x * 8; i < V; i += blockDim.x * 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(x + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float z[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      z[2 * e] = capf(f.x, cap) * inv_t;
      z[2 * e + 1] = capf(f.y, cap) * inv_t;
    }
    float zm = z[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) zm = fmaxf(zm, z[e]);
    if (zm > m) {
      s *= __expf(m - zm);
      m = zm;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) s += __expf(z[e] - m);
  }
  const float gm = block_max(m, red);
  const float part = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float tot = block_sum(part, red);
  if (threadIdx.x == 0) {
    const float l = gm + logf(tot);
    const long long t = targets[row];
    const float zt = (t >= 0 && t < V) ? capf(__bfloat162float(x[t]), cap) * inv_t : -INFINITY;
    lp[row] = zt - l;
    lse[row] = l;
  }
}

__global__ void logprob_rows_bwd_vec_kernel(__nv_bfloat16* __restrict__ logits, long long ld,
                                            const long long* __restrict__ targets, const float* __restrict__ lse,
                                            const float* __restrict__ dlp, int V, float inv_t, float cap) {
  const long long row = blockIdx.x;
  __nv_bfloat16* x = logits + row * ld;
  const float l = lse[row], g = dlp[row];
  const long long t = targets[row];
  for (int i = threadIdx.x * 8; i < V; i += blockDim.x * 8) {
    uint4 raw = *reinterpret_cast<const uint4*>(x + i);
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      float d[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const float rawv = k == 0 ? f.x : f.y;
        const float y = capf(rawv, cap);
        const float p = __expf(y * inv_t - l);
        float dd = g * (((i + 2 * e + k) == t ? 1.f : 0.f) - p) * inv_t;
        if (cap > 0.f) {
          const float th = y / cap;
          dd *= (1.f - th * th);
        }
        d[k] = dd;
      }
      h[e] = __floats2bfloat162_rn(d[0], d[1]);
    }
    *reinterpret_cast<uint4*>(x + i) = raw;
  }
}

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

constexpr int ST = 1024;  // threads per row

// VEC (16-bit logits, V a multiple of 8, 16-byte aligned rows): a thread takes 8 consecutive logits
// per 16-byte load, so every pass keeps eight times the bytes in flight; the passes are bound by
// L2 latency and the histograms and integer sums do not depend on the element order.
template <typename T, bool VEC>
__global__ void __launch_bounds__(ST)
sample_rows_kernel(const T* __restrict__ logits, long long ld, const long long* __restrict__ global_rows,
                   uint64_t seed, const int* __restrict__ draw_dev, int draw_host, long long* __restrict__ tok_out,
                   float* __restrict__ lp_out, int V, float inv_t, float top_p) {
  __shared__ float red[32];
  __shared__ unsigned long long hist[256];
  __shared__ unsigned long long sh_u64[4];
  __shared__ unsigned int sh_u32[2];
  // dynamic (96 KB): 32 warp-private histograms of three planes of 256 u32; the first 8 KB double as the
  // scan array afterwards
  extern __shared__ __align__(16) unsigned long long dyn[];
  unsigned long long* scan = dyn;
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  const int tid = threadIdx.x;
  const float FIX = 1099511627776.f;  // 2^40

  // Every pass over the row is bound by L2 latency, not bandwidth: a thread issues UL loads (of one
  // element, or of a group of eight) before anything consumes them.
  constexpr int EPT = VEC ? 8 : 1;          // elements per load
  constexpr int UL = VEC ? 2 : 4;           // loads in flight per thread
  constexpr int NV = UL * EPT;
  const int Vg = V / EPT;                   // groups in the row (VEC: V % 8 == 0)
  auto load_group = [&](int g, float* v) {  // group g -> EPT values (-inf past the end)
    if (VEC) {
      if (g < Vg) {
        const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + static_cast<long long>(g) * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(h[k]);
          v[2 * k] = f.x;
          v[2 * k + 1] = f.y;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = -INFINITY;
      }
    } else {
      v[0] = g < V ? to_f(x[g]) : -INFINITY;
    }
  };
  auto load_batch = [&](int g0, float* v) {
#pragma unroll
    for (int u = 0; u < UL; ++u) load_group(g0 + u * ST, v + u * EPT);
  };
  float m = -INFINITY;
  for (int i0 = tid; i0 < Vg; i0 += UL * ST) {
    float v[NV];
    load_batch(i0, v);
#pragma unroll
    for (int u = 0; u < NV; ++u) m = fmaxf(m, v[u]);
  }
  m = block_max(m, red);

  auto e_val = [&](float xv) -> float { return __expf((xv - m) * inv_t); };   // exp(-inf) = 0 for padding lanes
  auto fix_of = [&](float e) -> unsigned long long { return static_cast<unsigned long long>(e * FIX); };

  // Radix keys.  For 16-bit logits the order of the probabilities is the order of the logits, so the
  // nucleus cut is found on the sortable 16-bit pattern of the logit itself: two 8-bit passes instead
  // of four over the fp32 probability, and the first histogram also yields the total mass.
  constexpr bool K16 = sizeof(T) == 2;
  constexpr int N_PASS = K16 ? 2 : 4;
  auto key_of = [&](float xv, float e) -> unsigned int {
    if (K16) {
      const unsigned int u = __float_as_uint(xv) >> 16;
      return (u & 0x8000u) ? (~u & 0xFFFFu) : (u | 0x8000u);
    }
    return __float_as_uint(e);
  };
  const bool nucleus = top_p > 0.f && top_p < 1.f;

  // total mass (taken from the first histogram instead when that is built anyway)
  if (tid == 0) sh_u64[0] = 0;
  __syncthreads();
  if (!(K16 && nucleus)) {
    unsigned long long part = 0;
    for (int i0 = tid; i0 < Vg; i0 += UL * ST) {
      float v[NV];
      load_batch(i0, v);
#pragma unroll
      for (int u = 0; u < NV; ++u) part += fix_of(e_val(v[u]));
    }
    // warp-level integer reduction, then one atomic per warp
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if ((tid & 31) == 0) atomicAdd(&sh_u64[0], part);
  }
  __syncthreads();
  unsigned long long Z = sh_u64[0];

  unsigned int thresh_key = 0;          // keep everything
  unsigned long long kept_mass = Z;
  if (nucleus) {
    unsigned long long target =
        static_cast<unsigned long long>(static_cast<double>(Z) * static_cast<double>(top_p));
    unsigned int prefix = 0;
    unsigned long long above = 0;
    for (int pass = 0; pass < N_PASS; ++pass) {
      const int shift = 8 * (N_PASS - 1 - pass);
      for (int i = tid; i < 32 * 3 * 128; i += ST) dyn[i] = 0;     // 32 warps x 3 planes of 256 u32
      __syncthreads();
      // Each warp fills its own histogram with native 32-bit shared atomics on 14/13/13-bit pieces of the
      // fixed-point mass (a 64-bit shared atomic is a compare-and-swap loop; integer sums stay
      // order-independent).  A thread first adds up runs of equal buckets in registers: in the first
      // pass the digit is the sign and the high exponent bits, so runs are long and atomics few.
      {
        unsigned int* planes = reinterpret_cast<unsigned int*>(dyn) + (threadIdx.x >> 5) * 3 * 256;
        unsigned int cb = 0xFFFFFFFFu;
        unsigned long long cf = 0;
        auto flush = [&]() {
          if (cb != 0xFFFFFFFFu && cf) {
            atomicAdd(&planes[cb], static_cast<unsigned int>(cf & 0x3FFFu));
            atomicAdd(&planes[256 + cb], static_cast<unsigned int>((cf >> 14) & 0x1FFFu));
            atomicAdd(&planes[512 + cb], static_cast<unsigned int>(cf >> 27));
          }
        };
        for (int ib = 0; ib < Vg; ib += UL * ST) {
          float xv[NV];
          load_batch(ib + tid, xv);
#pragma unroll
          for (int u = 0; u < NV; ++u) {
            const float e = e_val(xv[u]);          // lanes past the end hold -inf: zero mass, no bucket
            const unsigned int key = key_of(xv[u], e);
            if (pass == 0 || (key >> (shift + 8)) == prefix) {
              const unsigned long long f = fix_of(e);
              if (f) {
                const unsigned int bucket = (key >> shift) & 0xFF;
                if (bucket == cb) {
                  cf += f;
                } else {
                  flush();
                  cb = bucket;
                  cf = f;
                }
              }
            }
          }
        }
        flush();
      }
      __syncthreads();
      if (tid < 256) {
        unsigned long long t = 0;
        const unsigned int* planes = reinterpret_cast<const unsigned int*>(dyn);
        for (int w = 0; w < 32; ++w)
          t += static_cast<unsigned long long>(planes[(w * 3) * 256 + tid]) +
               (static_cast<unsigned long long>(planes[(w * 3 + 1) * 256 + tid]) << 14) +
               (static_cast<unsigned long long>(planes[(w * 3 + 2) * 256 + tid]) << 27);
        hist[tid] = t;
      }
      __syncthreads();
      if (tid == 0) {
        if (K16 && pass == 0) {          // the first histogram covers every element: its sum is the total mass
          unsigned long long z = 0;
          for (int b = 0; b < 256; ++b) z += hist[b];
          sh_u64[0] = z;
          sh_u64[3] = static_cast<unsigned long long>(static_cast<double>(z) * static_cast<double>(top_p));
        }
        const unsigned long long target_ = (K16 && pass == 0) ? sh_u64[3] : target;
        unsigned long long cum = above;
        int b = 255;
        for (; b > 0; --b) {
          if (hist[b] > 0 && cum + hist[b] >= target_) break;
          cum += hist[b];
        }
        sh_u64[1] = cum;                 // mass strictly above the chosen bucket
        sh_u64[2] = cum + hist[b];       // mass of chosen bucket and above
        sh_u32[0] = (prefix << 8) | static_cast<unsigned int>(b);
      }
      __syncthreads();
      above = sh_u64[1];
      kept_mass = sh_u64[2];
      prefix = sh_u32[0];
      if (K16 && pass == 0) {
        Z = sh_u64[0];
        target = sh_u64[3];
      }
      __syncthreads();
    }
    thresh_key = prefix;
  }

  // draw
  const int draw = draw_dev ? *draw_dev : draw_host;
  const uint64_t key = mix64(seed + static_cast<uint64_t>(global_rows[row]) * 0x9E3779B97F4A7C15ull);
  const uint64_t bits = mix64(key + static_cast<uint64_t>(draw + 1) * 0x9E3779B97F4A7C15ull);
  const unsigned long long u24 = bits >> 40;
  const unsigned long long target = (kept_mass >> 24) * u24 + (((kept_mass & 0xFFFFFFull) * u24) >> 24);

  // contiguous chunk per thread, block scan of chunk masses, then the owning thread walks its chunk
  const int chunk = (Vg + ST - 1) / ST;                 // groups per thread
  const int c0 = tid * chunk, c1 = min(Vg, c0 + chunk);
  unsigned long long mine = 0;
  for (int g = c0; g < c1; ++g) {
    float xg[EPT];
    load_group(g, xg);
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      const float e = e_val(xg[k]);
      if (key_of(xg[k], e) >= thresh_key) mine += fix_of(e);
    }
  }
  __syncthreads();
  scan[tid] = mine;
  __syncthreads();
  // Hillis-Steele inclusive scan (1024 entries, 10 steps)
  for (int off = 1; off < ST; off <<= 1) {
    unsigned long long v = (tid >= off) ? scan[tid - off] : 0;
    __syncthreads();
    scan[tid] += v;
    __syncthreads();
  }
  const unsigned long long incl = scan[tid], excl = incl - mine;
  if (tid == 0) sh_u32[1] = 0xFFFFFFFFu;
  __syncthreads();
  if (mine > 0 && target >= excl && target < incl) {
    unsigned long long cum = excl;
    int pick = c1 * EPT - 1;
    bool found = false;
    for (int g = c0; g < c1 && !found; ++g) {
      float xg[EPT];
      load_group(g, xg);
#pragma unroll
      for (int k = 0; k < EPT; ++k) {
        const float e = e_val(xg[k]);
        if (!found && key_of(xg[k], e) >= thresh_key) {
          cum += fix_of(e);
          if (cum > target) {
            pick = g * EPT + k;
            found = true;
          }
        }
      }
    }
    sh_u32[1] = static_cast<unsigned int>(pick);
  }
  __syncthreads();
  if (tid == 0) {
    unsigned int pick = sh_u32[1];
    if (pick == 0xFFFFFFFFu) {
      // degenerate row (all mass rounded to zero): fall back to the arg-max element
      pick = 0;
      float best = -INFINITY;
      for (int i = 0; i < V; ++i) {
        float v = to_f(x[i]);
        if (v > best) { best = v; pick = i; }
      }
    }
    tok_out[row] = pick;
    float le = (to_f(x[pick]) - m) * inv_t;
    float lmass = logf(static_cast<float>(static_cast<double>(kept_mass) / 1099511627776.0));
    lp_out[row] = fminf(le - lmass, 0.f);
  }
}

}  // namespace

// Combine the per-tile (max, sum exp) pairs of the head GEMM's log-prob epilogue: lse = log sum exp over the
// vocabulary, lp = target logit - lse.  One thread per row; the tile-major layout keeps the reads coalesced.
__global__ void logprob_finalize_kernel(const float2* __restrict__ ws, const float* __restrict__ tl, int n_tiles, int M,
                                        float* __restrict__ lp, float* __restrict__ lse) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float m = -INFINITY;
  for (int t = 0; t < n_tiles; ++t) m = fmaxf(m, ws[static_cast<long long>(t) * M + row].x);
  float s = 0.f;
  for (int t = 0; t < n_tiles; ++t) {
    const float2 v = ws[static_cast<long long>(t) * M + row];
    s += v.y * __expf(v.x - m);
  }
  const float l = m + __logf(s);
  lse[row] = l;
  lp[row] = tl[row] - l;
}

// Vocabulary-sharded form: the same combine, but the result stays a partial (max, sum exp, target logit) per row,
// to be merged with the other shards' partials (tensor-parallel head).  stats [M, 3].
__global__ void logprob_shard_stats_kernel(const float2* __restrict__ ws, const float* __restrict__ tl, int n_tiles, int M,
                                           float* __restrict__ stats) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= M) return;
  float m = -INFINITY;
  for (int t = 0; t < n_tiles; ++t) m = fmaxf(m, ws[static_cast<long long>(t) * M + row].x);
  float s = 0.f;
  for (int t = 0; t < n_tiles; ++t) {
    const float2 v = ws[static_cast<long long>(t) * M + row];
    s += v.y * __expf(v.x - m);
  }
  stats[3 * row] = m;
  stats[3 * row + 1] = s;
  stats[3 * row + 2] = tl[row];
}

const char* logprob_shard_stats(const float* ws, const float* tl, int n_tiles, int M, float* stats, cudaStream_t s) {
  if (M == 0) return nullptr;
  logprob_shard_stats_kernel<<<(M + 127) / 128, 128, 0, s>>>(reinterpret_cast<const float2*>(ws), tl, n_tiles, M, stats);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "logprob_shard_stats launch failed";
}

const char* logprob_finalize(const float* ws, const float* tl, int n_tiles, int M, float* lp, float* lse, cudaStream_t s) {
  if (M == 0) return nullptr;
  logprob_finalize_kernel<<<(M + 127) / 128, 128, 0, s>>>(reinterpret_cast<const float2*>(ws), tl, n_tiles, M, lp, lse);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "logprob_finalize launch failed";
}

const char* logprob_rows(int dtype, const void* logits, long long ld, const long long* targets, float* lp, float* lse,
                         long long rows, int V, float temperature, float softcap, cudaStream_t s) {
  if (rows == 0) return nullptr;
  float inv_t = 1.f / temperature;
  if (dtype == kF32)
    logprob_rows_kernel<float><<<static_cast<unsigned>(rows), 1024, 0, s>>>(static_cast<const float*>(logits), ld,
                                                                           targets, lp, lse, V, inv_t, softcap);
  else if ((V % 8) == 0 && (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0)
    logprob_rows_vec_kernel<<<static_cast<unsigned>(rows), 512, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), ld,
                                                                       targets, lp, lse, V, inv_t, softcap);
  else
    logprob_rows_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), 1024, 0, s>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, targets, lp, lse, V, inv_t, softcap);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "logprob_rows launch failed";
}

const char* logprob_rows_bwd(int dtype, void* logits, long long ld, const long long* targets, const float* lse,
                             const float* dlp, long long rows, int V, float temperature, float softcap,
                             cudaStream_t s) {
  if (rows == 0) return nullptr;
  float inv_t = 1.f / temperature;
  if (dtype == kF32)
    logprob_rows_bwd_kernel<float><<<static_cast<unsigned>(rows), 1024, 0, s>>>(static_cast<float*>(logits), ld,
                                                                               targets, lse, dlp, V, inv_t, softcap);
  else if ((V % 8) == 0 && (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0)
    logprob_rows_bwd_vec_kernel<<<static_cast<unsigned>(rows), 512, 0, s>>>(static_cast<__nv_bfloat16*>(logits), ld,
                                                                           targets, lse, dlp, V, inv_t, softcap);
  else
    logprob_rows_bwd_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), 1024, 0, s>>>(
        static_cast<__nv_bfloat16*>(logits), ld, targets, lse, dlp, V, inv_t, softcap);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "logprob_rows_bwd launch failed";
}

const char* sample_rows(int dtype, const void* logits, long long ld, const long long* global_rows,
                        unsigned long long seed, const int* draw_dev, int draw_host, long long* tok_out, float* lp_out,
                        int rows, int V, float temperature, float top_p, cudaStream_t s) {
  if (rows == 0) return nullptr;
  float inv_t = 1.f / temperature;
  constexpr size_t kDyn = 32 * 3 * 128 * sizeof(unsigned long long);   // 96 KB: see the histogram passes
  if (!FERRL_ONCE_PER_DEVICE(
          cudaFuncSetAttribute(sample_rows_kernel<float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kDyn)) == cudaSuccess &&
          cudaFuncSetAttribute(sample_rows_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kDyn)) == cudaSuccess &&
          cudaFuncSetAttribute(sample_rows_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kDyn)) == cudaSuccess))
    return "sample_rows: cannot reserve shared memory";
  if (dtype == kF32)
    sample_rows_kernel<float, false><<<rows, ST, kDyn, s>>>(static_cast<const float*>(logits), ld, global_rows, seed, draw_dev,
                                                         draw_host, tok_out, lp_out, V, inv_t, top_p);
  else if ((V % 8) == 0 && (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0)
    sample_rows_kernel<__nv_bfloat16, true><<<rows, ST, kDyn, s>>>(static_cast<const __nv_bfloat16*>(logits), ld, global_rows,
                                                                seed, draw_dev, draw_host, tok_out, lp_out, V, inv_t, top_p);
  else
    sample_rows_kernel<__nv_bfloat16, false><<<rows, ST, kDyn, s>>>(static_cast<const __nv_bfloat16*>(logits), ld, global_rows,
                                                                 seed, draw_dev, draw_host, tok_out, lp_out, V, inv_t, top_p);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "sample_rows launch failed";
}

}  // namespace ferrl
