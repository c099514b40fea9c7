// KV-cached decode attention for sm_100a (bf16 cache, fp32 math), GQA-native.
//
// One CTA handles one (sequence, kv-head, kv-split): the `rep = Hq/Hkv` query heads that share
// the kv head are processed together, so every K and V row is read from HBM exactly once per
// step (the reference repeats the whole cache per query head and re-allocates it per token).
// K rows are consumed lane-per-key (each lane streams one 2*D-byte row with 16-byte loads, q is
// broadcast from shared memory); V rows are consumed warp-per-key (coalesced) with the key's
// probabilities broadcast by shuffle.  Online softmax per warp, warps merged through shared
// memory, kv-splits merged by a second tiny kernel through a caller-provided workspace.
// Supports a sliding window (keys older than `window` are skipped without being read) and a
// page table (`block_table[b, j / page]` gives the physical page of logical key j).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"

namespace ferrl {
namespace {

constexpr int WARPS = 4;
constexpr int MAX_REP = 8;
constexpr int MAX_DPL = 8;  // dims per lane: D <= 256

__global__ void __launch_bounds__(WARPS * 32)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                   const __nv_bfloat16* __restrict__ vc, const int* __restrict__ kv_len,
                   const int* __restrict__ block_table, int bt_stride, int page, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ ws, int Hq, int Hkv, int D, long long seq_stride, long long tok_stride,
                   float scale, int window, int n_splits) {
  pdl_trigger();   // a dependent GEMM may start streaming its weights while this kernel runs
  pdl_wait();      // launched as a programmatic dependent itself: nothing is read before the predecessor is done
  extern __shared__ float sm[];
  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int rep = Hq / Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dpl = (D + 31) / 32;
  float* q_s = sm;                               // [rep][D]
  float* m_s = q_s + rep * D;                    // [WARPS][rep]
  float* l_s = m_s + WARPS * rep;                // [WARPS][rep]
  float* o_s = l_s + WARPS * rep;                // [WARPS][rep][D]

  for (int i = threadIdx.x; i < rep * D; i += blockDim.x) {
    int r = i / D, d = i - r * D;
    q_s[i] = __bfloat162float(q[(static_cast<long long>(b) * Hq + hk * rep + r) * D + d]) * scale;
  }
  __syncthreads();

  const int len = kv_len[b];
  int lo = (window > 0 && len > window) ? len - window : 0;
  // split the live range [lo, len) evenly
  const int span = len - lo;
  const int per = (span + n_splits - 1) / n_splits;
  const int s0 = lo + split * per;
  const int s1 = min(len, s0 + per);

  float m_run[MAX_REP], l_run[MAX_REP], o_acc[MAX_REP][MAX_DPL];
#pragma unroll
  for (int r = 0; r < MAX_REP; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_DPL; ++i) o_acc[r][i] = 0.f;
  }

  for (int base = s0 + warp * 32; base < s1; base += WARPS * 32) {
    const int j = base + lane;
    const bool live = j < s1;
    long long row = 0;
    if (live) {
      if (block_table) {
        int pg = block_table[static_cast<long long>(b) * bt_stride + j / page];
        row = (static_cast<long long>(pg) * page + (j % page)) * tok_stride + hk * D;
      } else {
        row = static_cast<long long>(b) * seq_stride + static_cast<long long>(j) * tok_stride + hk * D;
      }
    }
    float sc[MAX_REP];
#pragma unroll
    for (int r = 0; r < MAX_REP; ++r) sc[r] = 0.f;
    if (live) {
      const uint4* kp = reinterpret_cast<const uint4*>(kc + row);
      for (int d8 = 0; d8 < D / 8; ++d8) {
        uint4 x = kp[d8];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
        float kf[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = __bfloat1622float2(h[e]);
          kf[2 * e] = f.x;
          kf[2 * e + 1] = f.y;
        }
#pragma unroll
        for (int r = 0; r < MAX_REP; ++r) {
          if (r < rep) {
            const float* qr = q_s + r * D + d8 * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) sc[r] += kf[e] * qr[e];
          }
        }
      }
    }
    // online softmax update for this tile of up to 32 keys
    float p[MAX_REP];
#pragma unroll
    for (int r = 0; r < MAX_REP; ++r) {
      p[r] = 0.f;
      if (r < rep) {
        float s = live ? sc[r] : -INFINITY;
        float tmax = warp_max(s);
        float m_new = fmaxf(m_run[r], tmax);
        float corr = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - m_new);
        p[r] = live ? __expf(s - m_new) : 0.f;
        float psum = warp_sum(p[r]);
        l_run[r] = l_run[r] * corr + psum;
        m_run[r] = m_new;
#pragma unroll
        for (int i = 0; i < MAX_DPL; ++i) o_acc[r][i] *= corr;
      }
    }
    const int nk = min(32, s1 - base);
    for (int kk = 0; kk < nk; ++kk) {
      const long long vrow = __shfl_sync(0xffffffffu, row, kk);
      float vv[MAX_DPL];
#pragma unroll
      for (int i = 0; i < MAX_DPL; ++i) {
        int d = lane + 32 * i;
        vv[i] = (i < dpl && d < D) ? __bfloat162float(vc[vrow + d]) : 0.f;
      }
#pragma unroll
      for (int r = 0; r < MAX_REP; ++r) {
        if (r < rep) {
          float pj = __shfl_sync(0xffffffffu, p[r], kk);
#pragma unroll
          for (int i = 0; i < MAX_DPL; ++i) o_acc[r][i] += pj * vv[i];
        }
      }
    }
  }

  // merge warps
  for (int r = 0; r < rep; ++r) {
    if (lane == 0) {
      m_s[warp * rep + r] = m_run[r];
      l_s[warp * rep + r] = l_run[r];
    }
    for (int i = 0; i < dpl; ++i) {
      int d = lane + 32 * i;
      if (d < D) o_s[(warp * rep + r) * D + d] = o_acc[r][i];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < rep * D; i += blockDim.x) {
    int r = i / D, d = i - r * D;
    float m = -INFINITY;
    for (int w = 0; w < WARPS; ++w) m = fmaxf(m, m_s[w * rep + r]);
    float l = 0.f, o = 0.f;
    for (int w = 0; w < WARPS; ++w) {
      float mw = m_s[w * rep + r];
      float c = (mw == -INFINITY) ? 0.f : __expf(mw - m);
      l += l_s[w * rep + r] * c;
      o += o_s[(w * rep + r) * D + d] * c;
    }
    const long long head = static_cast<long long>(b) * Hq + hk * rep + r;
    if (n_splits == 1) {
      out[head * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    } else {
      float* w_ = ws + (head * n_splits + split) * (D + 2);
      w_[d] = o;
      if (d == 0) {
        w_[D] = m;
        w_[D + 1] = l;
      }
    }
  }
}

// Fast path for head_dim 64 / 128 / 256.  LPK = D/16 lanes cooperate on one key, each owning 16
// channels: q (all `rep` heads) and the output accumulators live in registers, K and V rows are
// read with two coalesced 16-byte loads per lane, and four keys per lane group are in flight at
// once (no shared memory in the loop).  Every lane group keeps its own running (max, sum, out)
// and the groups are merged once at the end: across groups by shuffle, across warps through
// shared memory, across kv-splits through the workspace.
template <int D, int REP>
__global__ void __launch_bounds__(WARPS * 32)
decode_attn_fast_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                        const __nv_bfloat16* __restrict__ vc, const int* __restrict__ kv_len,
                        const int* __restrict__ block_table, int bt_stride, int page,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ ws, int Hq, int Hkv,
                        long long seq_stride, long long tok_stride, float scale, int window, int n_splits) {
  pdl_trigger();   // a dependent GEMM may start streaming its weights while this kernel runs
  pdl_wait();      // launched as a programmatic dependent itself: nothing is read before the predecessor is done
  constexpr int LPK = D / 16;        // lanes per key
  constexpr int KPW = 32 / LPK;      // keys per warp per step
  constexpr int UNROLL = (REP >= 6) ? 2 : 4;   // key steps in flight (bounded by the register file)
  extern __shared__ float sm[];
  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LPK, grp = lane / LPK;
  const int d0 = sub * 16;

  float qr[REP][16];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    const __nv_bfloat16* qp = q + (static_cast<long long>(b) * Hq + hk * REP + r) * D + d0;
#pragma unroll
    for (int e = 0; e < 16; ++e) qr[r][e] = __bfloat162float(qp[e]) * scale;
  }
  const int len = kv_len[b];
  const int lo = (window > 0 && len > window) ? len - window : 0;
  const int span = len - lo;
  const int per = (span + n_splits - 1) / n_splits;
  const int s0 = lo + split * per;
  const int s1 = min(len, s0 + per);

  float m_run[REP], l_run[REP], o[REP][16];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) o[r][e] = 0.f;
  }

  auto row_of = [&](int j) -> long long {
    if (block_table) {
      int pg = block_table[static_cast<long long>(b) * bt_stride + j / page];
      return (static_cast<long long>(pg) * page + (j % page)) * tok_stride + hk * D + d0;
    }
    return static_cast<long long>(b) * seq_stride + static_cast<long long>(j) * tok_stride + hk * D + d0;
  };

  // The trip count must be the same for every lane of a warp (the score reduction below shuffles
  // across the full warp), so the loop runs on the warp's first key and lanes past the end idle.
  for (int wbase = s0 + warp * KPW; wbase < s1; wbase += WARPS * KPW * UNROLL) {
    const int base = wbase + grp;
    uint4 kraw[UNROLL][2], vraw[UNROLL][2];
    bool live[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int j = base + u * WARPS * KPW;
      live[u] = j < s1;
      const long long row = live[u] ? row_of(j) : row_of(s0);
      const uint4* kp = reinterpret_cast<const uint4*>(kc + row);
      const uint4* vp = reinterpret_cast<const uint4*>(vc + row);
      kraw[u][0] = kp[0]; kraw[u][1] = kp[1];
      vraw[u][0] = vp[0]; vraw[u][1] = vp[1];
    }
    float sc[UNROLL][REP];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float kf[16];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&kraw[u][0]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float2 f = __bfloat1622float2(h[e]);
        kf[2 * e] = f.x;
        kf[2 * e + 1] = f.y;
      }
#pragma unroll
      for (int r = 0; r < REP; ++r) {
        float a = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) a += kf[e] * qr[r][e];
#pragma unroll
        for (int off = LPK / 2; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        sc[u][r] = live[u] ? a : -INFINITY;
      }
    }
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float mx = m_run[r];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) mx = fmaxf(mx, sc[u][r]);
      const float corr = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - mx);
      m_run[r] = mx;
      l_run[r] *= corr;
#pragma unroll
      for (int e = 0; e < 16; ++e) o[r][e] *= corr;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const float pj = (sc[u][r] == -INFINITY) ? 0.f : __expf(sc[u][r] - mx);
        sc[u][r] = pj;
        l_run[r] += pj;
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float vf[16];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&vraw[u][0]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float2 f = __bfloat1622float2(h[e]);
        vf[2 * e] = f.x;
        vf[2 * e + 1] = f.y;
      }
#pragma unroll
      for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int e = 0; e < 16; ++e) o[r][e] += sc[u][r] * vf[e];
    }
  }

  // merge the lane groups of this warp (same channels, different keys)
#pragma unroll
  for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m_run[r], off);
      const float l2 = __shfl_xor_sync(0xffffffffu, l_run[r], off);
      const float mn = fmaxf(m_run[r], m2);
      const float c1 = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - mn);
      const float c2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
      l_run[r] = l_run[r] * c1 + l2 * c2;
      m_run[r] = mn;
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const float o2 = __shfl_xor_sync(0xffffffffu, o[r][e], off);
        o[r][e] = o[r][e] * c1 + o2 * c2;
      }
    }
  }
  // merge warps through shared memory
  float* m_s = sm;                          // [WARPS][REP]
  float* l_s = m_s + WARPS * REP;           // [WARPS][REP]
  float* o_s = l_s + WARPS * REP;           // [WARPS][REP][D]
  if (grp == 0) {
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      if (sub == 0) {
        m_s[warp * REP + r] = m_run[r];
        l_s[warp * REP + r] = l_run[r];
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) o_s[(warp * REP + r) * D + d0 + e] = o[r][e];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < REP * D; i += blockDim.x) {
    const int r = i / D, d = i - r * D;
    float m = -INFINITY;
    for (int w = 0; w < WARPS; ++w) m = fmaxf(m, m_s[w * REP + r]);
    float l = 0.f, acc = 0.f;
    for (int w = 0; w < WARPS; ++w) {
      const float mw = m_s[w * REP + r];
      const float c = (mw == -INFINITY) ? 0.f : __expf(mw - m);
      l += l_s[w * REP + r] * c;
      acc += o_s[(w * REP + r) * D + d] * c;
    }
    const long long head = static_cast<long long>(b) * Hq + hk * REP + r;
    if (n_splits == 1) {
      out[head * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      float* w_ = ws + (head * n_splits + split) * (D + 2);
      w_[d] = acc;
      if (d == 0) {
        w_[D] = m;
        w_[D + 1] = l;
      }
    }
  }
}

// Shared-memory pipelined variant.  K/V rows stream through a ring of cp.async stages so the bytes
// in flight per SM no longer depend on the register file: a CTA of 4 warps keeps 3 stages of
// 32 keys (K and V) outstanding and three CTAs fit on an SM.  The math is the register-resident
// scheme above, reading its 32-byte key slices from shared memory (a quarter-warp reads whole
// 128-byte lines, so there are no bank conflicts).
constexpr int PWARPS = 4;
constexpr int PTK = 32;       // keys per stage
constexpr int PSTAGES = 4;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  const int n = valid ? 16 : 0;   // zero-fill when the key is past the end
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int D, int REP>
__global__ void __launch_bounds__(PWARPS * 32)
decode_attn_pipe_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                        const __nv_bfloat16* __restrict__ vc, const int* __restrict__ kv_len,
                        const int* __restrict__ block_table, int bt_stride, int page,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ ws, int Hq, int Hkv,
                        long long seq_stride, long long tok_stride, float scale, int window, int n_splits) {
  pdl_trigger();   // a dependent GEMM may start streaming its weights while this kernel runs
  pdl_wait();      // launched as a programmatic dependent itself: nothing is read before the predecessor is done
  constexpr int LPK = D / 16;                 // lanes per key
  constexpr int KPW = 32 / LPK;               // keys per warp per step
  constexpr int STEPS = PTK / (PWARPS * KPW); // steps per stage
  static_assert(STEPS >= 1, "tile too small for this head dim");
  constexpr int ROW_BYTES = D * 2;
  constexpr int CHUNKS = PTK * ROW_BYTES / 16;          // 16-byte chunks per K (or V) tile
  constexpr int STAGE_BYTES = 2 * PTK * ROW_BYTES;
  extern __shared__ __align__(128) uint8_t psm[];
  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LPK, grp = lane / LPK;
  const int d0 = sub * 16;

  float qr[REP][16];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    const __nv_bfloat16* qp = q + (static_cast<long long>(b) * Hq + hk * REP + r) * D + d0;
#pragma unroll
    for (int e = 0; e < 16; ++e) qr[r][e] = __bfloat162float(qp[e]) * scale;
  }
  const int len = kv_len[b];
  const int lo = (window > 0 && len > window) ? len - window : 0;
  const int span = len - lo;
  const int per = (span + n_splits - 1) / n_splits;
  const int s0 = lo + split * per;
  const int s1 = min(len, s0 + per);
  const int n_tiles = s1 > s0 ? (s1 - s0 + PTK - 1) / PTK : 0;

  auto row_of = [&](int j) -> long long {
    if (block_table) {
      int pg = block_table[static_cast<long long>(b) * bt_stride + j / page];
      return (static_cast<long long>(pg) * page + (j % page)) * tok_stride + hk * D;
    }
    return static_cast<long long>(b) * seq_stride + static_cast<long long>(j) * tok_stride + hk * D;
  };
  auto issue = [&](int t) {
    if (t < n_tiles) {
      uint8_t* st = psm + (t % PSTAGES) * STAGE_BYTES;
      const int j0 = s0 + t * PTK;
      for (int c = threadIdx.x; c < CHUNKS; c += PWARPS * 32) {
        const int key = c / (ROW_BYTES / 16), part = c % (ROW_BYTES / 16);
        const int j = j0 + key;
        const bool ok = j < s1;
        const long long row = row_of(ok ? j : s0) + part * 8;
        cp_async16(st + c * 16, kc + row, ok);
        cp_async16(st + PTK * ROW_BYTES + c * 16, vc + row, ok);
      }
    }
    cp_async_commit();     // one group per tile slot, empty past the end, so the wait count stays fixed
  };

  float m_run[REP], l_run[REP], o[REP][16];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    m_run[r] = -INFINITY;
    l_run[r] = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) o[r][e] = 0.f;
  }

#pragma unroll
  for (int t = 0; t < PSTAGES - 1; ++t) issue(t);
  for (int t = 0; t < n_tiles; ++t) {
    cp_async_wait<PSTAGES - 2>();
    __syncthreads();                 // tile t has landed for everyone; tile t-1's stage is free again
    issue(t + PSTAGES - 1);
    const uint8_t* st = psm + (t % PSTAGES) * STAGE_BYTES;
    const int j0 = s0 + t * PTK;
    float sc[STEPS][REP];
#pragma unroll
    for (int u = 0; u < STEPS; ++u) {
      const int kt = u * (PWARPS * KPW) + warp * KPW + grp;
      const bool live = j0 + kt < s1;
      const uint4* kp = reinterpret_cast<const uint4*>(st + kt * ROW_BYTES + d0 * 2);
      const uint4 k0 = kp[0], k1 = kp[1];
      float kf[16];
      const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&k0);
      const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&k1);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(h0[e]);
        kf[2 * e] = f.x;
        kf[2 * e + 1] = f.y;
        f = __bfloat1622float2(h1[e]);
        kf[8 + 2 * e] = f.x;
        kf[8 + 2 * e + 1] = f.y;
      }
#pragma unroll
      for (int r = 0; r < REP; ++r) {
        float a = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) a += kf[e] * qr[r][e];
#pragma unroll
        for (int off = LPK / 2; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        sc[u][r] = live ? a : -INFINITY;
      }
    }
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float mx = m_run[r];
#pragma unroll
      for (int u = 0; u < STEPS; ++u) mx = fmaxf(mx, sc[u][r]);
      const float corr = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - mx);
      m_run[r] = mx;
      l_run[r] *= corr;
#pragma unroll
      for (int e = 0; e < 16; ++e) o[r][e] *= corr;
#pragma unroll
      for (int u = 0; u < STEPS; ++u) {
        const float pj = (sc[u][r] == -INFINITY) ? 0.f : __expf(sc[u][r] - mx);
        sc[u][r] = pj;
        l_run[r] += pj;
      }
    }
#pragma unroll
    for (int u = 0; u < STEPS; ++u) {
      const int kt = u * (PWARPS * KPW) + warp * KPW + grp;
      const uint4* vp = reinterpret_cast<const uint4*>(st + PTK * ROW_BYTES + kt * ROW_BYTES + d0 * 2);
      const uint4 v0 = vp[0], v1 = vp[1];
      float vf[16];
      const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&v0);
      const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&v1);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(h0[e]);
        vf[2 * e] = f.x;
        vf[2 * e + 1] = f.y;
        f = __bfloat1622float2(h1[e]);
        vf[8 + 2 * e] = f.x;
        vf[8 + 2 * e + 1] = f.y;
      }
#pragma unroll
      for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int e = 0; e < 16; ++e) o[r][e] += sc[u][r] * vf[e];
    }
  }
  cp_async_wait<0>();
  __syncthreads();                   // the ring is reused below for the cross-warp merge

  // merge the lane groups of this warp (same channels, different keys)
#pragma unroll
  for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m_run[r], off);
      const float l2 = __shfl_xor_sync(0xffffffffu, l_run[r], off);
      const float mn = fmaxf(m_run[r], m2);
      const float c1 = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - mn);
      const float c2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
      l_run[r] = l_run[r] * c1 + l2 * c2;
      m_run[r] = mn;
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const float o2 = __shfl_xor_sync(0xffffffffu, o[r][e], off);
        o[r][e] = o[r][e] * c1 + o2 * c2;
      }
    }
  }
  float* m_s = reinterpret_cast<float*>(psm);   // [PWARPS][REP]
  float* l_s = m_s + PWARPS * REP;              // [PWARPS][REP]
  float* o_s = l_s + PWARPS * REP;              // [PWARPS][REP][D]
  if (grp == 0) {
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      if (sub == 0) {
        m_s[warp * REP + r] = m_run[r];
        l_s[warp * REP + r] = l_run[r];
      }
#pragma unroll
      for (int e = 0; e < 16; ++e) o_s[(warp * REP + r) * D + d0 + e] = o[r][e];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < REP * D; i += blockDim.x) {
    const int r = i / D, d = i - r * D;
    float m = -INFINITY;
    for (int w = 0; w < PWARPS; ++w) m = fmaxf(m, m_s[w * REP + r]);
    float l = 0.f, acc = 0.f;
    for (int w = 0; w < PWARPS; ++w) {
      const float mw = m_s[w * REP + r];
      const float c = (mw == -INFINITY) ? 0.f : __expf(mw - m);
      l += l_s[w * REP + r] * c;
      acc += o_s[(w * REP + r) * D + d] * c;
    }
    const long long head = static_cast<long long>(b) * Hq + hk * REP + r;
    if (n_splits == 1) {
      out[head * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      float* w_ = ws + (head * n_splits + split) * (D + 2);
      w_[d] = acc;
      if (d == 0) {
        w_[D] = m;
        w_[D + 1] = l;
      }
    }
  }
}

// Tensor-core variant of the pipelined kernel.  The query heads that share a KV head are the M
// dimension of the MMA (rows 0..REP-1 of a 16-row tile, the rest zero): scores S = Q K^T run on
// mma.sync m16n8k16 with K fragments out of ldmatrix, P V on m16n8k8 with the P fragment taken
// straight from the score accumulators and V fragments out of ldmatrix.trans.  Each warp owns 8 of
// the 32 keys of a stage and keeps its own running max / sum / output; warps are merged at the end.
// This removes the fp32 dot products from the CUDA cores, which bound the scalar kernel at ~57 %
// of HBM bandwidth.  Shared-memory rows are XOR-swizzled by 16-byte chunk.
__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_1688(float* c, uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// Three stages of 32 keys (48 KB at head_dim 128) let four CTAs share an SM: 592 CTA slots take the
// 1024 (row, kv-head) items of a 128-row batch in two waves instead of three.
constexpr int MSTAGES = 3;

template <int D, int REP>
__global__ void __launch_bounds__(PWARPS * 32, (D <= 128 && REP <= 4) ? 4 : 1)
decode_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                       const __nv_bfloat16* __restrict__ vc, const int* __restrict__ kv_len,
                       const int* __restrict__ block_table, int bt_stride, int page,
                       __nv_bfloat16* __restrict__ out, float* __restrict__ ws, int Hq, int Hkv,
                       long long seq_stride, long long tok_stride, float scale, int window, int n_splits,
                       const int* __restrict__ kv_start, int kv_start_div, int ws_off, int ws_total) {
  pdl_trigger();   // a dependent GEMM may start streaming its weights while this kernel runs
  pdl_wait();      // launched as a programmatic dependent itself: nothing is read before the predecessor is done
  static_assert(REP <= 8, "query heads of one KV head must fit rows 0..7 of the MMA tile");
  constexpr int ROW_BYTES = D * 2;
  constexpr int CPR = ROW_BYTES / 16;                  // 16-byte chunks per row
  constexpr int CHUNKS = PTK * CPR;
  constexpr int STAGE_BYTES = 2 * PTK * ROW_BYTES;
  constexpr int KSTEPS = D / 16;
  constexpr int NT = D / 8;                            // output n-tiles
  extern __shared__ __align__(128) uint8_t psm[];
  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  // Q fragments: rows g < REP are query heads hk*REP + g; a1 = a3 = 0 (rows 8..15 unused)
  uint32_t qa0[KSTEPS], qa2[KSTEPS];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    qa0[ks] = 0u;
    qa2[ks] = 0u;
    if (g < REP) {
      const __nv_bfloat16* qp = q + (static_cast<long long>(b) * Hq + hk * REP + g) * D + ks * 16 + 2 * t;
      qa0[ks] = *reinterpret_cast<const uint32_t*>(qp);
      qa2[ks] = *reinterpret_cast<const uint32_t*>(qp + 8);
    }
  }
  const int len = kv_len[b];
  int lo = (window > 0 && len > window) ? len - window : 0;
  // keys below kv_start[b / kv_start_div] belong to a prefix that another kernel covers (see the group kernel)
  if (kv_start) lo = max(lo, kv_start[b / kv_start_div]);
  const int span = max(len - lo, 0);
  const int per = (span + n_splits - 1) / n_splits;
  const int s0 = lo + split * per;
  const int s1 = min(len, s0 + per);
  const int n_tiles = s1 > s0 ? (s1 - s0 + PTK - 1) / PTK : 0;

  auto row_of = [&](int j) -> long long {
    if (block_table) {
      int pg = block_table[static_cast<long long>(b) * bt_stride + j / page];
      return (static_cast<long long>(pg) * page + (j % page)) * tok_stride + hk * D;
    }
    return static_cast<long long>(b) * seq_stride + static_cast<long long>(j) * tok_stride + hk * D;
  };
  auto issue = [&](int tt) {
    if (tt < n_tiles) {
      uint8_t* st = psm + (tt % MSTAGES) * STAGE_BYTES;
      const int j0 = s0 + tt * PTK;
      for (int c = threadIdx.x; c < CHUNKS; c += PWARPS * 32) {
        const int key = c / CPR, part = c % CPR;
        const int j = j0 + key;
        const bool ok = j < s1;
        const long long row = row_of(ok ? j : s0) + part * 8;
        const int off = key * ROW_BYTES + ((part ^ (key & 7)) << 4);
        cp_async16(st + off, kc + row, ok);
        cp_async16(st + PTK * ROW_BYTES + off, vc + row, ok);
      }
    }
    cp_async_commit();
  };

  float m_run = -INFINITY, l_run = 0.f;     // row g of this warp's keys
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

#pragma unroll
  for (int tt = 0; tt < MSTAGES - 1; ++tt) issue(tt);
  for (int tt = 0; tt < n_tiles; ++tt) {
    cp_async_wait<MSTAGES - 2>();
    __syncthreads();
    issue(tt + MSTAGES - 1);
    const uint32_t kt = static_cast<uint32_t>(__cvta_generic_to_shared(psm + (tt % MSTAGES) * STAGE_BYTES));
    const uint32_t vt = kt + PTK * ROW_BYTES;
    const int key0 = warp * 8;                        // this warp's 8 keys of the tile
    const int j0 = s0 + tt * PTK + key0;
    // ---- S = Q K^T for 8 keys
    float sacc[4] = {0.f, 0.f, 0.f, 0.f};
    const int lrow = key0 + (lane & 7), lmat = lane >> 3;
#pragma unroll
    for (int qd = 0; qd < KSTEPS / 2; ++qd) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4(kt + lrow * ROW_BYTES + (((4 * qd + lmat) ^ (lrow & 7)) << 4), b0, b1, b2, b3);
      mma_16816(sacc, qa0[2 * qd], 0u, qa2[2 * qd], 0u, b0, b1);
      mma_16816(sacc, qa0[2 * qd + 1], 0u, qa2[2 * qd + 1], 0u, b2, b3);
    }
    // ---- online softmax on row g over keys (2t, 2t+1) of the 4 lanes sharing g
    float sc0 = (j0 + 2 * t < s1) ? sacc[0] * scale : -INFINITY;
    float sc1 = (j0 + 2 * t + 1 < s1) ? sacc[1] * scale : -INFINITY;
    float mx = fmaxf(sc0, sc1);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float corr = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_new);
    const float p0 = (sc0 == -INFINITY) ? 0.f : __expf(sc0 - m_new);
    const float p1 = (sc1 == -INFINITY) ? 0.f : __expf(sc1 - m_new);
    float ps = p0 + p1;
    ps += __shfl_xor_sync(0xffffffffu, ps, 1);
    ps += __shfl_xor_sync(0xffffffffu, ps, 2);
    l_run = l_run * corr + ps;
    m_run = m_new;
    __nv_bfloat162 ph = __floats2bfloat162_rn(p0, p1);
    const uint32_t pa0 = *reinterpret_cast<uint32_t*>(&ph);
    // ---- O = O * corr + P V
#pragma unroll
    for (int qd = 0; qd < NT / 4; ++qd) {
      uint32_t v0, v1, v2, v3;
      ldsm_x4_t(vt + lrow * ROW_BYTES + (((4 * qd + lmat) ^ (lrow & 7)) << 4), v0, v1, v2, v3);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o[4 * qd + e][0] *= corr;
        o[4 * qd + e][1] *= corr;
      }
      mma_1688(o[4 * qd + 0], pa0, 0u, v0);
      mma_1688(o[4 * qd + 1], pa0, 0u, v1);
      mma_1688(o[4 * qd + 2], pa0, 0u, v2);
      mma_1688(o[4 * qd + 3], pa0, 0u, v3);
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge warps through shared memory (the ring is free now)
  float* m_s = reinterpret_cast<float*>(psm);   // [PWARPS][REP]
  float* l_s = m_s + PWARPS * REP;              // [PWARPS][REP]
  float* o_s = l_s + PWARPS * REP;              // [PWARPS][REP][D]
  if (g < REP) {
    if (t == 0) {
      m_s[warp * REP + g] = m_run;
      l_s[warp * REP + g] = l_run;
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o_s[(warp * REP + g) * D + n * 8 + 2 * t] = o[n][0];
      o_s[(warp * REP + g) * D + n * 8 + 2 * t + 1] = o[n][1];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < REP * D; i += blockDim.x) {
    const int r = i / D, d = i - r * D;
    float m = -INFINITY;
    for (int w = 0; w < PWARPS; ++w) m = fmaxf(m, m_s[w * REP + r]);
    float l = 0.f, acc = 0.f;
    for (int w = 0; w < PWARPS; ++w) {
      const float mw = m_s[w * REP + r];
      const float c = (mw == -INFINITY) ? 0.f : __expf(mw - m);
      l += l_s[w * REP + r] * c;
      acc += o_s[(w * REP + r) * D + d] * c;
    }
    const long long head = static_cast<long long>(b) * Hq + hk * REP + r;
    if (ws_total > 0) {
      // shared-prefix mode: merge my keys with the prefix partials and write the final row
      const float* base = ws + head * ws_total * (D + 2);
      float mm = m;
      for (int sp = 0; sp < ws_off; ++sp) mm = fmaxf(mm, base[sp * (D + 2) + D]);
      const float c0 = (m == -INFINITY) ? 0.f : __expf(m - mm);
      float lt = l * c0, ot = acc * c0;
      for (int sp = 0; sp < ws_off; ++sp) {
        const float ms = base[sp * (D + 2) + D];
        const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
        lt += base[sp * (D + 2) + D + 1] * c;
        ot += base[sp * (D + 2) + d] * c;
      }
      out[head * D + d] = __float2bfloat16_rn((lt > 0.f && len > 0) ? ot / lt : 0.f);   // a retired row (length 0) stays zero
    } else if (n_splits == 1) {
      out[head * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      float* w_ = ws + (head * n_splits + split) * (D + 2);
      w_[d] = acc;
      if (d == 0) {
        w_[D] = m;
        w_[D + 1] = l;
      }
    }
  }
}

// Shared-prefix form for grouped rollouts.  The G rows of a group (one prompt, G completions) share
// the prompt's full pages, so the keys [0, prefix_len[group]) are the same memory for all of them: one
// CTA per (group, KV head, split) streams those keys ONCE and applies them to all G * REP query rows
// of the group (two 16-row MMA tiles for G = 8, REP = 4) instead of G CTAs streaming them G times.
// The rest of every row ([prefix_len, kv_len)) is covered by decode_attn_mma_kernel with kv_start =
// prefix_len, launched right behind this kernel as its programmatic dependent; in its last step it merges
// the (o, m, l) partials written here with its own and writes the final rows (no combine kernel).
// Query row r of the tile is batch row group * G + r / REP, head hk * REP + r % REP.
// Eight warps for 32 query rows: warp w takes keys 8 (w & 3) .. +7 of every 32-key tile for the 16-row MMA tile
// w >> 2, so two warps share each scheduler and two CTAs (four ring stages each) fit an SM.
constexpr int GSTAGES = 4;

template <int D, int REP, int G>
__global__ void __launch_bounds__(PWARPS * 32 * (REP * G / 16), 2)
decode_attn_group_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                         const __nv_bfloat16* __restrict__ vc, const int* __restrict__ prefix_len,
                         const int* __restrict__ kv_len, const int* __restrict__ block_table, int bt_stride, int page,
                         float* __restrict__ ws, int Hq, int Hkv, long long tok_stride, float scale, int n_splits,
                         int ws_total) {
  pdl_trigger();   // the per-row kernel may take its place on the SMs; it waits for this kernel before it reads anything
  pdl_wait();
  constexpr int QR = REP * G;                          // query rows sharing the keys
  static_assert(QR % 16 == 0 && QR <= 32, "group kernel: G * REP must be 16 or 32");
  constexpr int ROW_BYTES = D * 2;
  constexpr int CPR = ROW_BYTES / 16;
  constexpr int CHUNKS = PTK * CPR;
  constexpr int STAGE_BYTES = 2 * PTK * ROW_BYTES;
  constexpr int KSTEPS = D / 16;
  constexpr int NT = D / 8;
  extern __shared__ __align__(128) uint8_t psm[];
  const int gi = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kq = warp & 3, rt = warp >> 2;             // key octet of the tile, 16-row tile of the queries
  const int g = lane >> 2, t = lane & 3;

  int pre = prefix_len[gi];
  {
    // a group whose rows have all been retired (attention length 0) reads nothing
    int live = 0;
    for (int r = 0; r < G; ++r) live |= kv_len[gi * G + r];
    if (live == 0) pre = 0;
  }
  const int per = (pre + n_splits - 1) / n_splits;
  const int s0 = split * per;
  const int s1 = min(pre, s0 + per);
  const int n_tiles = s1 > s0 ? (s1 - s0 + PTK - 1) / PTK : 0;
  const int b0 = gi * G;                               // the group's first row: its table names the shared pages

  // Q fragments of my row tile: rows rt*16 + g (a0, a2) and rt*16 + g + 8 (a1, a3)
  uint32_t qa[KSTEPS][4];
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = rt * 16 + g + 8 * hh;
    const __nv_bfloat16* qp = q + (static_cast<long long>(b0 + r / REP) * Hq + hk * REP + r % REP) * D + 2 * t;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      qa[ks][hh] = *reinterpret_cast<const uint32_t*>(qp + ks * 16);
      qa[ks][2 + hh] = *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8);
    }
  }

  auto row_of = [&](int j) -> long long {
    const int pg = block_table[static_cast<long long>(b0) * bt_stride + j / page];
    return (static_cast<long long>(pg) * page + (j % page)) * tok_stride + hk * D;
  };
  auto issue = [&](int tt) {
    if (tt < n_tiles) {
      uint8_t* st = psm + (tt % GSTAGES) * STAGE_BYTES;
      const int j0 = s0 + tt * PTK;
      for (int c = threadIdx.x; c < CHUNKS; c += blockDim.x) {
        const int key = c / CPR, part = c % CPR;
        const int j = j0 + key;
        const bool ok = j < s1;
        const long long row = row_of(ok ? j : s0) + part * 8;
        const int off = key * ROW_BYTES + ((part ^ (key & 7)) << 4);
        cp_async16(st + off, kc + row, ok);
        cp_async16(st + PTK * ROW_BYTES + off, vc + row, ok);
      }
    }
    cp_async_commit();
  };

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

#pragma unroll
  for (int tt = 0; tt < GSTAGES - 1; ++tt) issue(tt);
  for (int tt = 0; tt < n_tiles; ++tt) {
    cp_async_wait<GSTAGES - 2>();
    __syncthreads();
    issue(tt + GSTAGES - 1);
    const uint32_t kt = static_cast<uint32_t>(__cvta_generic_to_shared(psm + (tt % GSTAGES) * STAGE_BYTES));
    const uint32_t vt = kt + PTK * ROW_BYTES;
    const int key0 = kq * 8;
    const int j0 = s0 + tt * PTK + key0;
    const int lrow = key0 + (lane & 7), lmat = lane >> 3;
    float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int qd = 0; qd < KSTEPS / 2; ++qd) {
      uint32_t b0_, b1_, b2_, b3_;
      ldsm_x4(kt + lrow * ROW_BYTES + (((4 * qd + lmat) ^ (lrow & 7)) << 4), b0_, b1_, b2_, b3_);
      mma_16816(sacc, qa[2 * qd][0], qa[2 * qd][1], qa[2 * qd][2], qa[2 * qd][3], b0_, b1_);
      mma_16816(sacc, qa[2 * qd + 1][0], qa[2 * qd + 1][1], qa[2 * qd + 1][2], qa[2 * qd + 1][3], b2_, b3_);
    }
    const bool v0 = j0 + 2 * t < s1, v1 = j0 + 2 * t + 1 < s1;
    uint32_t pa[2];
    float corr[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const float sc0 = v0 ? sacc[2 * hh] * scale : -INFINITY;
      const float sc1 = v1 ? sacc[2 * hh + 1] * scale : -INFINITY;
      float mx = fmaxf(sc0, sc1);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hh], mx);
      const float cr = (m_run[hh] == -INFINITY) ? 0.f : __expf(m_run[hh] - m_new);
      const float p0 = (sc0 == -INFINITY) ? 0.f : __expf(sc0 - m_new);
      const float p1 = (sc1 == -INFINITY) ? 0.f : __expf(sc1 - m_new);
      float ps = p0 + p1;
      ps += __shfl_xor_sync(0xffffffffu, ps, 1);
      ps += __shfl_xor_sync(0xffffffffu, ps, 2);
      l_run[hh] = l_run[hh] * cr + ps;
      m_run[hh] = m_new;
      corr[hh] = cr;
      __nv_bfloat162 ph = __floats2bfloat162_rn(p0, p1);
      pa[hh] = *reinterpret_cast<uint32_t*>(&ph);
    }
#pragma unroll
    for (int qd = 0; qd < NT / 4; ++qd) {
      uint32_t w0, w1, w2, w3;
      ldsm_x4_t(vt + lrow * ROW_BYTES + (((4 * qd + lmat) ^ (lrow & 7)) << 4), w0, w1, w2, w3);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o[4 * qd + e][0] *= corr[0];
        o[4 * qd + e][1] *= corr[0];
        o[4 * qd + e][2] *= corr[1];
        o[4 * qd + e][3] *= corr[1];
      }
      mma_1688(o[4 * qd + 0], pa[0], pa[1], w0);
      mma_1688(o[4 * qd + 1], pa[0], pa[1], w1);
      mma_1688(o[4 * qd + 2], pa[0], pa[1], w2);
      mma_1688(o[4 * qd + 3], pa[0], pa[1], w3);
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the four key octets of every row through shared memory
  float* m_s = reinterpret_cast<float*>(psm);   // [4][QR]
  float* l_s = m_s + PWARPS * QR;               // [4][QR]
  float* o_s = l_s + PWARPS * QR;               // [4][QR][D]
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int r = rt * 16 + g + 8 * hh;
    if (t == 0) {
      m_s[kq * QR + r] = m_run[hh];
      l_s[kq * QR + r] = l_run[hh];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o_s[(kq * QR + r) * D + n * 8 + 2 * t] = o[n][2 * hh];
      o_s[(kq * QR + r) * D + n * 8 + 2 * t + 1] = o[n][2 * hh + 1];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < QR * D; i += blockDim.x) {
    const int r = i / D, d = i - r * D;
    float m = -INFINITY;
    for (int w = 0; w < PWARPS; ++w) m = fmaxf(m, m_s[w * QR + r]);
    float l = 0.f, acc = 0.f;
    for (int w = 0; w < PWARPS; ++w) {
      const float mw = m_s[w * QR + r];
      const float c = (mw == -INFINITY) ? 0.f : __expf(mw - m);
      l += l_s[w * QR + r] * c;
      acc += o_s[(w * QR + r) * D + d] * c;
    }
    const long long head = static_cast<long long>(b0 + r / REP) * Hq + hk * REP + r % REP;
    float* w_ = ws + (head * ws_total + split) * (D + 2);
    w_[d] = acc;
    if (d == 0) {
      w_[D] = m;
      w_[D + 1] = l;
    }
  }
}

// Whole-group form (D = 128, REP = 4, G = 8): one CTA per (group, KV head) does the shared prefix AND the
// private keys of the group's eight rows, so nothing crosses a kernel boundary (no workspace, no second
// launch, no dependency edge).
//   phase 1: the prefix keys stream once through a CTA-wide ring; all 32 query rows of the group (8 rows x 4
//            heads, two 16-row MMA tiles) are applied to them as in decode_attn_group_kernel; the four key
//            octets are merged into one (o, m, l) per query row in shared memory.
//   phase 2: warp w owns row w of the group: it streams that row's private keys [prefix_len, kv_len) through
//            its own 3-stage ring of 16 keys (no CTA-wide barrier in the loop), its 4 query heads being rows
//            0..3 of the MMA tile, then merges with the prefix partial of those heads and writes the row.
// Eight warps with 16 KB in flight each keep 128 KB of loads outstanding per SM.
constexpr int FSTAGES = 3;       // per-warp ring stages
constexpr int FKEYS = 16;        // keys per per-warp stage

__global__ void __launch_bounds__(256, 1)
decode_attn_group_fused_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                               const __nv_bfloat16* __restrict__ vc, const int* __restrict__ prefix_len,
                               const int* __restrict__ kv_len, const int* __restrict__ block_table, int bt_stride, int page,
                               __nv_bfloat16* __restrict__ out, int Hq, int Hkv, long long tok_stride, float scale) {
  pdl_trigger();
  pdl_wait();
  constexpr int D = 128, REP = 4, G = 8, QR = 32;
  constexpr int ROW_BYTES = D * 2;
  constexpr int CPR = ROW_BYTES / 16;
  constexpr int KSTEPS = D / 16;
  constexpr int NT = D / 8;
  constexpr int P1_STAGE = 2 * PTK * ROW_BYTES;            // 16 KB
  constexpr int W_STAGE = 2 * FKEYS * ROW_BYTES;           // 8 KB
  constexpr int RING_BYTES = 8 * FSTAGES * W_STAGE;        // 192 KB (phase 1 uses its first GSTAGES * 16 KB)
  extern __shared__ __align__(128) uint8_t psm[];
  float* pre_m = reinterpret_cast<float*>(psm + RING_BYTES);   // [32]
  float* pre_l = pre_m + QR;                                    // [32]
  float* pre_o = pre_l + QR;                                    // [32][128]
  const int gi = blockIdx.x, hk = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int b0 = gi * G;

  int pre = prefix_len[gi];
  {
    int live = 0;
    for (int r = 0; r < G; ++r) live |= kv_len[b0 + r];
    if (live == 0) pre = 0;
  }

  // ------------------------------------------------------------------ phase 1: shared prefix
  {
    const int kq = warp & 3, rt = warp >> 2;
    const int n_tiles = (pre + PTK - 1) / PTK;
    uint32_t qa[KSTEPS][4];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = rt * 16 + g + 8 * hh;
      const __nv_bfloat16* qp = q + (static_cast<long long>(b0 + r / REP) * Hq + hk * REP + r % REP) * D + 2 * t;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        qa[ks][hh] = *reinterpret_cast<const uint32_t*>(qp + ks * 16);
        qa[ks][2 + hh] = *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8);
      }
    }
    auto issue = [&](int tt) {
      if (tt < n_tiles) {
        uint8_t* st = psm + (tt % GSTAGES) * P1_STAGE;
        const int j0 = tt * PTK;
        for (int c = threadIdx.x; c < PTK * CPR; c += 256) {
          const int key = c / CPR, part = c % CPR;
          const int j = j0 + key;
          const bool ok = j < pre;
          const int jj = ok ? j : 0;
          const int pg = block_table[static_cast<long long>(b0) * bt_stride + jj / page];
          const long long row = (static_cast<long long>(pg) * page + (jj % page)) * tok_stride + hk * D + part * 8;
          const int off = key * ROW_BYTES + ((part ^ (key & 7)) << 4);
          cp_async16(st + off, kc + row, ok);
          cp_async16(st + PTK * ROW_BYTES + off, vc + row, ok);
        }
      }
      cp_async_commit();
    };
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
#pragma unroll
    for (int tt = 0; tt < GSTAGES - 1; ++tt) issue(tt);
    for (int tt = 0; tt < n_tiles; ++tt) {
      cp_async_wait<GSTAGES - 2>();
      __syncthreads();
      issue(tt + GSTAGES - 1);
      const uint32_t kt = static_cast<uint32_t>(__cvta_generic_to_shared(psm + (tt % GSTAGES) * P1_STAGE));
      const uint32_t vt = kt + PTK * ROW_BYTES;
      const int key0 = kq * 8;
      const int j0 = tt * PTK + key0;
      const int lrow = key0 + (lane & 7), lmat = lane >> 3;
      float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int qd = 0; qd < KSTEPS / 2; ++qd) {
        uint32_t b0_, b1_, b2_, b3_;
        ldsm_x4(kt + lrow * ROW_BYTES + (((4 * qd + lmat) ^ (lrow & 7)) << 4), b0_, b1_, b2_, b3_);
        mma_16816(sacc, qa[2 * qd][0], qa[2 * qd][1], qa[2 * qd][2], qa[2 * qd][3], b0_, b1_);
        mma_16816(sacc, qa[2 * qd + 1][0], qa[2 * qd + 1][1], qa[2 * qd + 1][2], qa[2 * qd + 1][3], b2_, b3_);
      }
      const bool v0 = j0 + 2 * t < pre, v1 = j0 + 2 * t + 1 < pre;
      uint32_t pa[2];
      float corr[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const float sc0 = v0 ? sacc[2 * hh] * scale : -INFINITY;
        const float sc1 = v1 ? sacc[2 * hh + 1] * scale : -INFINITY;
        float mx = fmaxf(sc0, sc1);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[hh], mx);
        const float cr = (m_run[hh] == -INFINITY) ? 0.f : __expf(m_run[hh] - m_new);
        const float p0 = (sc0 == -INFINITY) ? 0.f : __expf(sc0 - m_new);
        const float p1 = (sc1 == -INFINITY) ? 0.f : __expf(sc1 - m_new);
        float ps = p0 + p1;
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run[hh] = l_run[hh] * cr + ps;
        m_run[hh] = m_new;
        corr[hh] = cr;
        __nv_bfloat162 ph = __floats2bfloat162_rn(p0, p1);
        pa[hh] = *reinterpret_cast<uint32_t*>(&ph);
      }
#pragma unroll
      for (int qd = 0; qd < NT / 4; ++qd) {
        uint32_t w0, w1, w2, w3;
        ldsm_x4_t(vt + lrow * ROW_BYTES + (((4 * qd + lmat) ^ (lrow & 7)) << 4), w0, w1, w2, w3);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o[4 * qd + e][0] *= corr[0];
          o[4 * qd + e][1] *= corr[0];
          o[4 * qd + e][2] *= corr[1];
          o[4 * qd + e][3] *= corr[1];
        }
        mma_1688(o[4 * qd + 0], pa[0], pa[1], w0);
        mma_1688(o[4 * qd + 1], pa[0], pa[1], w1);
        mma_1688(o[4 * qd + 2], pa[0], pa[1], w2);
        mma_1688(o[4 * qd + 3], pa[0], pa[1], w3);
      }
    }
    cp_async_wait<0>();
    __syncthreads();
    // merge the four key octets of every query row: ring memory is free now
    float* m_s = reinterpret_cast<float*>(psm);   // [4][32]
    float* l_s = m_s + 4 * QR;
    float* o_s = l_s + 4 * QR;                    // [4][32][128]
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = rt * 16 + g + 8 * hh;
      if (t == 0) {
        m_s[kq * QR + r] = m_run[hh];
        l_s[kq * QR + r] = l_run[hh];
      }
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        o_s[(kq * QR + r) * D + n * 8 + 2 * t] = o[n][2 * hh];
        o_s[(kq * QR + r) * D + n * 8 + 2 * t + 1] = o[n][2 * hh + 1];
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < QR * D; i += 256) {
      const int r = i / D, d = i - r * D;
      float m = -INFINITY;
      for (int w = 0; w < 4; ++w) m = fmaxf(m, m_s[w * QR + r]);
      float l = 0.f, acc = 0.f;
      for (int w = 0; w < 4; ++w) {
        const float mw = m_s[w * QR + r];
        const float c = (mw == -INFINITY) ? 0.f : __expf(mw - m);
        l += l_s[w * QR + r] * c;
        acc += o_s[(w * QR + r) * D + d] * c;
      }
      pre_o[r * D + d] = acc;
      if (d == 0) {
        pre_m[r] = m;
        pre_l[r] = l;
      }
    }
    __syncthreads();
  }

  // ------------------------------------------------------------------ phase 2: warp w = row w of the group
  {
    const int b = b0 + warp;
    const int len = kv_len[b];
    const int lo = min(pre, len);
    const int n_tiles = len > lo ? (len - lo + FKEYS - 1) / FKEYS : 0;
    uint8_t* ring = psm + warp * (FSTAGES * W_STAGE);
    uint32_t qa0[KSTEPS], qa2[KSTEPS];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      qa0[ks] = 0u;
      qa2[ks] = 0u;
      if (g < REP) {
        const __nv_bfloat16* qp = q + (static_cast<long long>(b) * Hq + hk * REP + g) * D + ks * 16 + 2 * t;
        qa0[ks] = *reinterpret_cast<const uint32_t*>(qp);
        qa2[ks] = *reinterpret_cast<const uint32_t*>(qp + 8);
      }
    }
    auto issue = [&](int tt) {
      if (tt < n_tiles) {
        uint8_t* st = ring + (tt % FSTAGES) * W_STAGE;
        const int j0 = lo + tt * FKEYS;
        for (int c = lane; c < FKEYS * CPR; c += 32) {
          const int key = c / CPR, part = c % CPR;
          const int j = j0 + key;
          const bool ok = j < len;
          const int jj = ok ? j : lo;
          const int pg = block_table[static_cast<long long>(b) * bt_stride + jj / page];
          const long long row = (static_cast<long long>(pg) * page + (jj % page)) * tok_stride + hk * D + part * 8;
          const int off = key * ROW_BYTES + ((part ^ (key & 7)) << 4);
          cp_async16(st + off, kc + row, ok);
          cp_async16(st + FKEYS * ROW_BYTES + off, vc + row, ok);
        }
      }
      cp_async_commit();
    };
    float m_run = -INFINITY, l_run = 0.f;
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
#pragma unroll
    for (int tt = 0; tt < FSTAGES - 1; ++tt) issue(tt);
    for (int tt = 0; tt < n_tiles; ++tt) {
      cp_async_wait<FSTAGES - 2>();
      __syncwarp();
      issue(tt + FSTAGES - 1);
      const uint32_t kt = static_cast<uint32_t>(__cvta_generic_to_shared(ring + (tt % FSTAGES) * W_STAGE));
      const uint32_t vt = kt + FKEYS * ROW_BYTES;
#pragma unroll
      for (int oct = 0; oct < FKEYS / 8; ++oct) {
        const int key0 = oct * 8;
        const int j0 = lo + tt * FKEYS + key0;
        const int lrow = key0 + (lane & 7), lmat = lane >> 3;
        float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int qd = 0; qd < KSTEPS / 2; ++qd) {
          uint32_t b0_, b1_, b2_, b3_;
          ldsm_x4(kt + lrow * ROW_BYTES + (((4 * qd + lmat) ^ (lrow & 7)) << 4), b0_, b1_, b2_, b3_);
          mma_16816(sacc, qa0[2 * qd], 0u, qa2[2 * qd], 0u, b0_, b1_);
          mma_16816(sacc, qa0[2 * qd + 1], 0u, qa2[2 * qd + 1], 0u, b2_, b3_);
        }
        const float sc0 = (j0 + 2 * t < len) ? sacc[0] * scale : -INFINITY;
        const float sc1 = (j0 + 2 * t + 1 < len) ? sacc[1] * scale : -INFINITY;
        float mx = fmaxf(sc0, sc1);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float corr = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_new);
        const float p0 = (sc0 == -INFINITY) ? 0.f : __expf(sc0 - m_new);
        const float p1 = (sc1 == -INFINITY) ? 0.f : __expf(sc1 - m_new);
        float ps = p0 + p1;
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run = l_run * corr + ps;
        m_run = m_new;
        __nv_bfloat162 ph = __floats2bfloat162_rn(p0, p1);
        const uint32_t pa0 = *reinterpret_cast<uint32_t*>(&ph);
#pragma unroll
        for (int qd = 0; qd < NT / 4; ++qd) {
          uint32_t w0, w1, w2, w3;
          ldsm_x4_t(vt + lrow * ROW_BYTES + (((4 * qd + lmat) ^ (lrow & 7)) << 4), w0, w1, w2, w3);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            o[4 * qd + e][0] *= corr;
            o[4 * qd + e][1] *= corr;
          }
          mma_1688(o[4 * qd + 0], pa0, 0u, w0);
          mma_1688(o[4 * qd + 1], pa0, 0u, w1);
          mma_1688(o[4 * qd + 2], pa0, 0u, w2);
          mma_1688(o[4 * qd + 3], pa0, 0u, w3);
        }
      }
    }
    cp_async_wait<0>();
    // merge with the prefix partial of query row warp * 4 + g and write the row's 4 heads
    if (g < REP) {
      const int r = warp * REP + g;
      const float mp = pre_m[r], lp = pre_l[r];
      const float mm = fmaxf(m_run, mp);
      const float c0 = (m_run == -INFINITY) ? 0.f : __expf(m_run - mm);
      const float c1 = (mp == -INFINITY) ? 0.f : __expf(mp - mm);
      const float lt = l_run * c0 + lp * c1;
      const float inv = (lt > 0.f && len > 0) ? 1.f / lt : 0.f;           // a retired row (length 0) stays zero
      __nv_bfloat16* op = out + (static_cast<long long>(b) * Hq + hk * REP + g) * D;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int d = n * 8 + 2 * t;
        const float x0 = (o[n][0] * c0 + pre_o[r * D + d] * c1) * inv;
        const float x1 = (o[n][1] * c0 + pre_o[r * D + d + 1] * c1) * inv;
        *reinterpret_cast<__nv_bfloat162*>(op + d) = __floats2bfloat162_rn(x0, x1);
      }
    }
  }
}

__global__ void decode_combine_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, int D,
                                      int n_splits) {
  pdl_trigger();   // a dependent GEMM may start streaming its weights while this kernel runs
  pdl_wait();      // launched as a programmatic dependent itself: nothing is read before the predecessor is done
  const long long head = blockIdx.x;
  const float* base = ws + head * n_splits * (D + 2);
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, base[s * (D + 2) + D]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float l = 0.f, o = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      float ms = base[s * (D + 2) + D];
      float c = (ms == -INFINITY) ? 0.f : __expf(ms - m);
      l += base[s * (D + 2) + D + 1] * c;
      o += base[s * (D + 2) + d] * c;
    }
    out[head * D + d] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
  }
}

}  // namespace

size_t decode_attn_workspace_bytes(int B, int Hq, int D, int n_splits) {
  return n_splits <= 1 ? 0 : static_cast<size_t>(B) * Hq * n_splits * (D + 2) * sizeof(float);
}

int decode_attn_pick_splits(int B, int Hkv, int max_len, int num_sms) {
  long long ctas = static_cast<long long>(B) * Hkv;
  int s = 1;
  while (ctas * s < 2LL * num_sms && s < 16 && max_len / (s * 2) >= 256) s *= 2;
  return s;
}

const char* decode_attn(const DecodeAttnArgs& a, cudaStream_t s) {
  if (a.B == 0) return nullptr;
  if (a.Hq % a.Hkv) return "decode_attn: Hq must be a multiple of Hkv";
  const int rep = a.Hq / a.Hkv;
  if (rep > MAX_REP) return "decode_attn: more than 8 query heads per kv head";
  if (a.D % 8 || a.D > 256) return "decode_attn: head_dim must be a multiple of 8 and <= 256";
  if (a.n_splits > 1 && !a.workspace) return "decode_attn: workspace required for split-kv";
  dim3 grid(a.B, a.Hkv, a.n_splits < 1 ? 1 : a.n_splits);
  bool launched = false;
  // shared-prefix mode (grouped rollouts over a paged cache): see decode_attn_group_kernel
  const int* kv_start = nullptr;
  int kv_start_div = 1, ws_off = 0, ws_total = 0;
  if (a.prefix_len) {
    const int G = a.group;
    if (!a.block_table || !a.workspace || a.window > 0 || a.no_pipe != 0 || grid.z != 1 || G < 1 || (a.B % G) ||
        a.prefix_splits < 1 || a.prefix_splits > 8)
      return "decode_attn: shared-prefix mode needs a paged cache, a workspace, no window, one private split, 1..8 prefix splits";
    if ((a.tok_stride % 8) || (reinterpret_cast<uintptr_t>(a.k) & 15) || (reinterpret_cast<uintptr_t>(a.v) & 15) ||
        (reinterpret_cast<uintptr_t>(a.q) & 3))
      return "decode_attn: shared-prefix mode needs 16-byte aligned caches";
    if (a.D == 128 && rep == 4 && G == 8 && a.prefix_splits == 1) {
      // whole-group kernel: prefix and private keys in one launch, no workspace
      constexpr size_t fsm = static_cast<size_t>(8) * FSTAGES * 2 * FKEYS * 128 * 2 + (2 * 32 + 32 * 128) * 4;
      auto fk = decode_attn_group_fused_kernel;
      if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(fk, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      static_cast<int>(fsm)) == cudaSuccess))
        return "decode_attn: cannot reserve shared memory";
      launch_pdl(fk, dim3(a.B / 8, a.Hkv), dim3(256), fsm, s, static_cast<const __nv_bfloat16*>(a.q),
                 static_cast<const __nv_bfloat16*>(a.k), static_cast<const __nv_bfloat16*>(a.v), a.prefix_len, a.kv_len,
                 a.block_table, a.bt_stride, a.page, static_cast<__nv_bfloat16*>(a.out), a.Hq, a.Hkv, a.tok_stride, a.scale);
      count_launch();
      return cudaGetLastError() == cudaSuccess ? nullptr : "decode_attn launch failed";
    }
    kv_start = a.prefix_len; kv_start_div = G; ws_off = a.prefix_splits; ws_total = a.prefix_splits;
    bool ok = false;
#define FERRL_DECODE_GROUP(DD, RR, GG)                                                                                \
  if (!ok && a.D == DD && rep == RR && G == GG) {                                                                     \
    constexpr size_t ring = static_cast<size_t>(GSTAGES) * 2 * PTK * DD * 2;                                          \
    constexpr size_t merge = (2 * PWARPS * RR * GG + static_cast<size_t>(PWARPS) * RR * GG * DD) * 4;                 \
    constexpr size_t gsm = ring > merge ? ring : merge;                                                               \
    auto gk = decode_attn_group_kernel<DD, RR, GG>;                                                                   \
    if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(gk, cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                                                    static_cast<int>(gsm)) == cudaSuccess &&                          \
                               cudaFuncSetAttribute(gk, cudaFuncAttributePreferredSharedMemoryCarveout,               \
                                                    cudaSharedmemCarveoutMaxShared) == cudaSuccess))                  \
      return "decode_attn: cannot reserve shared memory";                                                             \
    launch_pdl(gk, dim3(a.B / GG, a.Hkv, a.prefix_splits), dim3(PWARPS * 32 * (RR * GG / 16)), gsm, s,                                 \
               static_cast<const __nv_bfloat16*>(a.q), static_cast<const __nv_bfloat16*>(a.k),                        \
               static_cast<const __nv_bfloat16*>(a.v), a.prefix_len, a.kv_len, a.block_table, a.bt_stride, a.page,    \
               a.workspace, a.Hq, a.Hkv, a.tok_stride, a.scale, a.prefix_splits, ws_total);                           \
    ok = true;                                                                                                        \
  }
    FERRL_DECODE_GROUP(128, 4, 8) FERRL_DECODE_GROUP(128, 4, 4) FERRL_DECODE_GROUP(128, 8, 4) FERRL_DECODE_GROUP(128, 8, 2)
    FERRL_DECODE_GROUP(128, 2, 8) FERRL_DECODE_GROUP(64, 4, 8) FERRL_DECODE_GROUP(64, 4, 4) FERRL_DECODE_GROUP(128, 2, 16)
#undef FERRL_DECODE_GROUP
    if (!ok) return "decode_attn: shared-prefix mode has no kernel for this (head_dim, heads per kv head, group) triple";
    count_launch();
  }
#define FERRL_DECODE_FAST(DD, RR)                                                                                   \
  if (!launched && a.D == DD && rep == RR && !kv_start) {                                                                          \
    size_t fsm = (2 * WARPS * RR + static_cast<size_t>(WARPS) * RR * DD) * 4;                                         \
    decode_attn_fast_kernel<DD, RR><<<grid, WARPS * 32, fsm, s>>>(                                                    \
        static_cast<const __nv_bfloat16*>(a.q), static_cast<const __nv_bfloat16*>(a.k),                               \
        static_cast<const __nv_bfloat16*>(a.v), a.kv_len, a.block_table, a.bt_stride, a.page,                         \
        static_cast<__nv_bfloat16*>(a.out), a.workspace, a.Hq, a.Hkv, a.seq_stride, a.tok_stride, a.scale, a.window,  \
        grid.z);                                                                                                      \
    launched = true;                                                                                                  \
  }
#define FERRL_DECODE_PIPE(DD, RR)                                                                                   \
  if (!launched && a.D == DD && rep == RR && a.no_pipe != 1 && !kv_start) {                                                            \
    constexpr size_t psm_bytes = static_cast<size_t>(PSTAGES) * 2 * PTK * DD * 2;                                     \
    auto pk = decode_attn_pipe_kernel<DD, RR>;                                                                        \
    if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                                                    static_cast<int>(psm_bytes)) == cudaSuccess))                     \
      return "decode_attn: cannot reserve shared memory";                                                             \
    pk<<<grid, PWARPS * 32, psm_bytes, s>>>(                                                                          \
        static_cast<const __nv_bfloat16*>(a.q), static_cast<const __nv_bfloat16*>(a.k),                               \
        static_cast<const __nv_bfloat16*>(a.v), a.kv_len, a.block_table, a.bt_stride, a.page,                         \
        static_cast<__nv_bfloat16*>(a.out), a.workspace, a.Hq, a.Hkv, a.seq_stride, a.tok_stride, a.scale, a.window,  \
        grid.z);                                                                                                      \
    launched = true;                                                                                                  \
  }
#define FERRL_DECODE_MMA(DD, RR)                                                                                    \
  if (!launched && a.D == DD && rep == RR && a.no_pipe == 0) {                                                        \
    constexpr size_t msm_bytes = static_cast<size_t>(MSTAGES) * 2 * PTK * DD * 2;                                     \
    auto mk = decode_attn_mma_kernel<DD, RR>;                                                                         \
    if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(mk, cudaFuncAttributeMaxDynamicSharedMemorySize,                  \
                                                    static_cast<int>(msm_bytes)) == cudaSuccess &&                    \
                               cudaFuncSetAttribute(mk, cudaFuncAttributePreferredSharedMemoryCarveout,               \
                                                    cudaSharedmemCarveoutMaxShared) == cudaSuccess))                  \
      return "decode_attn: cannot reserve shared memory";                                                             \
    launch_pdl(mk, grid, dim3(PWARPS * 32), msm_bytes, s,                                                             \
        static_cast<const __nv_bfloat16*>(a.q), static_cast<const __nv_bfloat16*>(a.k),                               \
        static_cast<const __nv_bfloat16*>(a.v), a.kv_len, a.block_table, a.bt_stride, a.page,                         \
        static_cast<__nv_bfloat16*>(a.out), a.workspace, a.Hq, a.Hkv, a.seq_stride, a.tok_stride, a.scale, a.window,  \
        grid.z, kv_start, kv_start_div, ws_off, ws_total);                                                            \
    launched = true;                                                                                                  \
  }
  if ((a.tok_stride % 8) == 0 && (a.seq_stride % 8) == 0 && (reinterpret_cast<uintptr_t>(a.k) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(a.v) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q) & 3) == 0) {
    FERRL_DECODE_MMA(128, 4) FERRL_DECODE_MMA(128, 1) FERRL_DECODE_MMA(128, 2) FERRL_DECODE_MMA(128, 8)
    FERRL_DECODE_MMA(64, 1) FERRL_DECODE_MMA(64, 2) FERRL_DECODE_MMA(64, 4) FERRL_DECODE_MMA(64, 8)
    FERRL_DECODE_MMA(256, 1) FERRL_DECODE_MMA(256, 2) FERRL_DECODE_MMA(256, 4) FERRL_DECODE_MMA(256, 6)
    FERRL_DECODE_MMA(256, 8)
  }
#undef FERRL_DECODE_MMA
  if ((a.tok_stride % 8) == 0 && (a.seq_stride % 8) == 0 && (reinterpret_cast<uintptr_t>(a.k) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(a.v) & 15) == 0) {
    FERRL_DECODE_PIPE(128, 4) FERRL_DECODE_PIPE(128, 1) FERRL_DECODE_PIPE(128, 2) FERRL_DECODE_PIPE(128, 8)
    FERRL_DECODE_PIPE(64, 1) FERRL_DECODE_PIPE(64, 2) FERRL_DECODE_PIPE(64, 4) FERRL_DECODE_PIPE(64, 8)
    FERRL_DECODE_PIPE(256, 1) FERRL_DECODE_PIPE(256, 2) FERRL_DECODE_PIPE(256, 4)
  }
#undef FERRL_DECODE_PIPE
  if ((a.tok_stride % 8) == 0 && (a.seq_stride % 8) == 0) {
    FERRL_DECODE_FAST(128, 4) FERRL_DECODE_FAST(128, 1) FERRL_DECODE_FAST(128, 2) FERRL_DECODE_FAST(128, 8)
    FERRL_DECODE_FAST(64, 1) FERRL_DECODE_FAST(64, 2) FERRL_DECODE_FAST(64, 4) FERRL_DECODE_FAST(64, 8)
    FERRL_DECODE_FAST(256, 1) FERRL_DECODE_FAST(256, 2) FERRL_DECODE_FAST(256, 4) FERRL_DECODE_FAST(256, 6)
    FERRL_DECODE_FAST(256, 8)
  }
#undef FERRL_DECODE_FAST
  if (!launched && kv_start) return "decode_attn: shared-prefix mode found no tensor-core kernel for the private part";
  if (!launched) {
    size_t smem = (static_cast<size_t>(rep) * a.D + 2 * WARPS * rep + static_cast<size_t>(WARPS) * rep * a.D) * 4;
    auto kern = decode_attn_kernel;
    if (smem > 48 * 1024) {
      if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) ==
                                 cudaSuccess))
        return "decode_attn: cannot reserve shared memory";
    }
    kern<<<grid, WARPS * 32, smem, s>>>(static_cast<const __nv_bfloat16*>(a.q), static_cast<const __nv_bfloat16*>(a.k),
                                        static_cast<const __nv_bfloat16*>(a.v), a.kv_len, a.block_table, a.bt_stride,
                                        a.page, static_cast<__nv_bfloat16*>(a.out), a.workspace, a.Hq, a.Hkv, a.D,
                                        a.seq_stride, a.tok_stride, a.scale, a.window, grid.z);
  }
  count_launch();
  if (grid.z > 1) {
    launch_pdl(decode_combine_kernel, dim3(a.B * a.Hq), dim3(128), 0, s, a.workspace, static_cast<__nv_bfloat16*>(a.out), a.D,
               static_cast<int>(grid.z));
    count_launch();
  }
  return cudaGetLastError() == cudaSuccess ? nullptr : "decode_attn launch failed";
}

}  // namespace ferrl

// ------------------------------------------------------------------------------------------------
// Allocation-free entry point (declared and documented in csrc/no_alloc.h).
#include <atomic>

#include "../no_alloc.h"

namespace {
// Split-KV workspace that lives in the library image: callers that may not allocate use this
// instead of a caller-provided buffer. In host code the name below is only a handle for
// cudaGetSymbolAddress - it is not a device address and must never be handed to a kernel.
static __device__ __align__(256) float g_static_decode_ws[FERRL_STATIC_WS_FLOATS];

constexpr int kMaxDevices = FERRL_NOALLOC_MAX_DEVICES;
// Written once per device with the same value by whichever host thread gets there first.
std::atomic<float*> g_static_ws_addr[kMaxDevices];
}  // namespace

extern "C" int ferrl_decode_attn_static_ws(const void* q, const void* k_cache, const void* v_cache, const int* kv_len,
                                           void* out, int B, int Hq, int Hkv, int D, long long seq_stride,
                                           long long tok_stride, float scale, int window, int n_splits, void* stream) {
  if (!q || !k_cache || !v_cache || !kv_len || !out || B < 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || n_splits < 1 ||
      n_splits > 16 || (Hq % Hkv) || (Hq / Hkv) > 8 || (D % 8) || D > 256 || window < 0 || seq_stride < 0 ||
      tok_stride < static_cast<long long>(Hkv) * D)
    return FERRL_NOALLOC_BAD_ARGS;
  if (B == 0) return FERRL_NOALLOC_OK;
  const unsigned long long need =
      n_splits > 1 ? static_cast<unsigned long long>(B) * Hq * n_splits * (D + 2) : 0ull;
  if (need > FERRL_STATIC_WS_FLOATS) return FERRL_NOALLOC_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FERRL_NOALLOC_CUDA_ERROR;
  float* ws = g_static_ws_addr[dev].load(std::memory_order_acquire);
  if (!ws) {
    // once per device, with that device current: turn the symbol into its device address
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ws), g_static_decode_ws) != cudaSuccess || !ws)
      return FERRL_NOALLOC_CUDA_ERROR;
    g_static_ws_addr[dev].store(ws, std::memory_order_release);
  }
  ferrl::DecodeAttnArgs a{};
  a.q = q; a.k = k_cache; a.v = v_cache; a.kv_len = kv_len; a.block_table = nullptr; a.bt_stride = 0; a.page = 0;
  a.out = out; a.workspace = n_splits > 1 ? ws : nullptr;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.seq_stride = seq_stride; a.tok_stride = tok_stride;
  a.scale = scale; a.window = window; a.n_splits = n_splits;
  return ferrl::decode_attn(a, static_cast<cudaStream_t>(stream)) == nullptr ? FERRL_NOALLOC_OK
                                                                             : FERRL_NOALLOC_CUDA_ERROR;
}

extern "C" const char* ferrl_noalloc_strerror(int code) {
  switch (code) {
    case FERRL_NOALLOC_OK: return "ok";
    case FERRL_NOALLOC_TOO_LARGE:
      return "B*Hq*n_splits*(D+2) exceeds the 4Mi-float static workspace; use fewer splits or a smaller batch";
    case FERRL_NOALLOC_BAD_ARGS:
      return "null pointer or unsupported geometry (need Hq%Hkv==0, Hq/Hkv<=8, D%8==0, D<=256, 1<=n_splits<=16, "
             "window>=0, seq_stride>=0, tok_stride>=Hkv*D)";
    case FERRL_NOALLOC_CUDA_ERROR:
      return "a CUDA call failed (device query, symbol address lookup or kernel launch), or the current device's "
             "ordinal is FERRL_NOALLOC_MAX_DEVICES or higher";
    default: return "unknown code";
  }
}
