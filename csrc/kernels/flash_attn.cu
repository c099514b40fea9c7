// Flash attention forward and backward (prefill / scoring / training), bf16, GQA-native.
//
// Causal and sliding-window masks are evaluated from indices inside the kernel (no mask
// tensors, no repeat_kv copies, nothing of size S^2 in memory); query i sits at absolute
// position q_offset + i.  q/k/v/o may be strided views (batch and token strides), so k and v
// are read straight out of the fused qkv projection buffer.
//
// Tiles: 64 queries x 64 keys per step, 4 warps x 16 query rows (forward, dQ) or 16 key rows
// (dK/dV).  Operands are staged with cp.async into XOR-swizzled shared memory and fed to
// mma.sync.m16n8k16 through ldmatrix.  Softmax runs in the exp2 domain with fp32 statistics.
// Backward is two deterministic passes (no atomics): dK/dV own a key block and sweep the
// query blocks of every query head in the kv group; dQ owns a query block and sweeps keys.
//
// The score and value contractions here still use the warp-level mma.sync path; the GEMMs
// around attention (95% of the FLOPs at these sequence lengths) are on tcgen05.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"

namespace ferrl {
namespace {

constexpr int BQ = 64;
constexpr int BKV = 64;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// byte offset of (row, 16-byte chunk) in a swizzled tile whose rows hold D bf16
template <int D>
__device__ __forceinline__ uint32_t sw_off(int row, int chunk) {
  return static_cast<uint32_t>(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Load a [64 x D] tile (rows row0.., limit n_rows) from a strided global tensor into swizzled smem.
template <int D, int THREADS>
__device__ __forceinline__ void load_tile(uint8_t* smem, const __nv_bfloat16* base, long long tok_stride, int row0,
                                          int n_rows) {
  constexpr int CH = D / 8;
  for (int i = threadIdx.x; i < 64 * CH; i += THREADS) {
    int r = i / CH, c = i - r * CH;
    bool ok = (row0 + r) < n_rows && (row0 + r) >= 0;
    const __nv_bfloat16* src = base + static_cast<long long>(ok ? row0 + r : 0) * tok_stride + c * 8;
    cp_async16(smem_u32(smem) + sw_off<D>(r, c), src, ok);
  }
}

// A fragment (16 x 16) of a row-major swizzled tile at rows r0.., k-chunk kk (16 columns)
template <int D>
__device__ __forceinline__ void load_a(const uint8_t* tile, int r0, int kk, uint32_t* a) {
  const int lane = threadIdx.x & 31;
  int row = r0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  int chunk = kk * 2 + (lane >> 4);
  ldsm4(smem_u32(tile) + sw_off<D>(row, chunk), a[0], a[1], a[2], a[3]);
}
// B fragments for two n-tiles (16 "n" rows n0..) from a tile stored [n][k], k-chunk kk
template <int D>
__device__ __forceinline__ void load_b_nk(const uint8_t* tile, int n0, int kk, uint32_t* b) {
  const int lane = threadIdx.x & 31;
  int row = n0 + (lane & 7) + (lane >> 4) * 8;
  int chunk = kk * 2 + ((lane >> 3) & 1);
  ldsm4(smem_u32(tile) + sw_off<D>(row, chunk), b[0], b[1], b[2], b[3]);
}
// B fragments for two n-tiles (16 columns n0..) from a tile stored [k][n], k rows k0..k0+15
template <int D>
__device__ __forceinline__ void load_b_kn(const uint8_t* tile, int k0, int n0, uint32_t* b) {
  const int lane = threadIdx.x & 31;
  int row = k0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  int chunk = (n0 >> 3) + (lane >> 4);
  ldsm4t(smem_u32(tile) + sw_off<D>(row, chunk), b[0], b[1], b[2], b[3]);
}

__device__ __forceinline__ bool allowed(int pos_i, int j, int Sk, int causal, int window) {
  return j < Sk && (!causal || j <= pos_i) && (window <= 0 || j > pos_i - window);
}

// --------------------------------------------------------------------------- forward
template <int D>
__global__ void __launch_bounds__(128) flash_fwd_kernel(FlashArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int TILE = 64 * D * 2;
  uint8_t* sQ = smem;
  uint8_t* sK[2] = {smem + TILE, smem + 3 * TILE};
  uint8_t* sV[2] = {smem + 2 * TILE, smem + 4 * TILE};
  const int m0 = blockIdx.x * BQ, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(a.q) + b * a.q_bs + h * D;
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(a.k) + b * a.k_bs + hk * D;
  const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(a.v) + b * a.v_bs + hk * D;

  int j_hi = a.causal ? min(a.Sk, a.q_offset + m0 + BQ) : a.Sk;
  int j_lo = a.window > 0 ? max(0, a.q_offset + m0 - a.window + 1) : 0;
  const int jb0 = j_lo / BKV, jb1 = (j_hi + BKV - 1) / BKV;

  load_tile<D, 128>(sQ, qb, a.q_ts, m0, a.Sq);
  if (jb0 < jb1) {
    load_tile<D, 128>(sK[0], kb, a.k_ts, jb0 * BKV, a.Sk);
    load_tile<D, 128>(sV[0], vb, a.v_ts, jb0 * BKV, a.Sk);
  }
  cp_commit();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float c = a.scale * LOG2E;
  const int r0 = warp * 16;
  const int pos0 = a.q_offset + m0 + r0 + g, pos1 = pos0 + 8;

  for (int jb = jb0; jb < jb1; ++jb) {
    const int buf = (jb - jb0) & 1;
    if (jb + 1 < jb1) {
      load_tile<D, 128>(sK[buf ^ 1], kb, a.k_ts, (jb + 1) * BKV, a.Sk);
      load_tile<D, 128>(sV[buf ^ 1], vb, a.v_ts, (jb + 1) * BKV, a.Sk);
    }
    cp_commit();
    cp_wait<1>();
    __syncthreads();

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t af[4];
      load_a<D>(sQ, r0, kk, af);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bf[4];
        load_b_nk<D>(sK[buf], np * 16, kk, bf);
        mma16816(s[2 * np], af, bf[0], bf[1]);
        mma16816(s[2 * np + 1], af, bf[2], bf[3]);
      }
    }
    // mask + row max
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int j = jb * BKV + nt * 8 + 2 * t + (e & 1);
        int pos = (e < 2) ? pos0 : pos1;
        if (!allowed(pos, j, a.Sk, a.causal, a.window)) s[nt][e] = -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
      corr[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f((m_run[r] - m_use[r]) * c);
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }
    uint32_t pf[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      float p0 = exp2f((s[nt][0] - m_use[0]) * c), p1 = exp2f((s[nt][1] - m_use[0]) * c);
      float p2 = exp2f((s[nt][2] - m_use[1]) * c), p3 = exp2f((s[nt][3] - m_use[1]) * c);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      pf[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
      pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int k2 = 0; k2 < 4; ++k2) {
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t bf[4];
        load_b_kn<D>(sV[buf], k2 * 16, dp * 16, bf);
        mma16816(o[2 * dp], pf[k2], bf[0], bf[1]);
        mma16816(o[2 * dp + 1], pf[k2], bf[2], bf[3]);
      }
    }
    __syncthreads();
  }
  cp_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  __nv_bfloat16* ob = static_cast<__nv_bfloat16*>(a.o) + b * a.o_bs + h * D;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    int row = m0 + r0 + g + r * 8;
    if (row >= a.Sq) continue;
    float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
    __nv_bfloat16* orow = ob + static_cast<long long>(row) * a.o_ts;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      *reinterpret_cast<uint32_t*>(orow + i * 8 + 2 * t) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
    if (t == 0 && a.lse)
      a.lse[(static_cast<long long>(b) * a.Hq + h) * a.Sq + row] =
          (l_run[r] > 0.f) ? m_run[r] * a.scale + logf(l_run[r]) : -INFINITY;
  }
}

// --------------------------------------------------------------------------- backward
__global__ void flash_delta_kernel(FlashArgs a) {
  // one warp per (b, i, h): delta = sum_d dO * O
  const long long wid = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(a.B) * a.Sq * a.Hq;
  if (wid >= total) return;
  const int h = static_cast<int>(wid % a.Hq);
  const long long bi = wid / a.Hq;
  const int i = static_cast<int>(bi % a.Sq), b = static_cast<int>(bi / a.Sq);
  const __nv_bfloat16* op = static_cast<const __nv_bfloat16*>(a.o) + b * a.o_bs + static_cast<long long>(i) * a.o_ts + h * a.D;
  const __nv_bfloat16* dp = static_cast<const __nv_bfloat16*>(a.d_o) + b * a.do_bs + static_cast<long long>(i) * a.do_ts + h * a.D;
  float s = 0.f;
  for (int d = lane; d < a.D; d += 32) s += __bfloat162float(op[d]) * __bfloat162float(dp[d]);
  s = warp_sum(s);
  if (lane == 0) a.delta[(static_cast<long long>(b) * a.Hq + h) * a.Sq + i] = s;
}

// dK/dV: CTA owns 64 keys of one kv head. DSPLIT warps groups split the head dim of the accumulators.
template <int D, int DSPLIT>
__global__ void __launch_bounds__(128 * DSPLIT) flash_bwd_dkv_kernel(FlashArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int TILE = 64 * D * 2;
  constexpr int THREADS = 128 * DSPLIT;
  constexpr int DW = D / DSPLIT;  // accumulator width per warp
  uint8_t* sK = smem;
  uint8_t* sV = smem + TILE;
  uint8_t* sQ = smem + 2 * TILE;
  uint8_t* sdO = smem + 3 * TILE;
  float* sLse = reinterpret_cast<float*>(smem + 4 * TILE);
  float* sDel = sLse + 64;
  const int n0 = blockIdx.x * BKV, hk = blockIdx.y, b = blockIdx.z;
  const int rep = a.Hq / a.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int kw = warp & 3, dh = warp >> 2;
  const int k0 = kw * 16, d0 = dh * DW;
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(a.k) + b * a.k_bs + hk * D;
  const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(a.v) + b * a.v_bs + hk * D;
  load_tile<D, THREADS>(sK, kb, a.k_ts, n0, a.Sk);
  load_tile<D, THREADS>(sV, vb, a.v_ts, n0, a.Sk);
  cp_commit();

  float dk[DW / 8][4], dv[DW / 8][4];
#pragma unroll
  for (int i = 0; i < DW / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
  }
  const float c = a.scale * LOG2E;
  // query rows that can see this key block: pos_i >= n0 (causal) and pos_i < n0 + 64 + window - 1
  int i_lo = a.causal ? max(0, n0 - a.q_offset) : 0;
  int i_hi = a.window > 0 ? min(a.Sq, n0 + BKV + a.window - 1 - a.q_offset) : a.Sq;
  const int ib0 = i_lo / BQ, ib1 = (i_hi + BQ - 1) / BQ;
  const int key0 = n0 + k0 + g, key1 = key0 + 8;

  for (int r = 0; r < rep; ++r) {
    const int h = hk * rep + r;
    const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(a.q) + b * a.q_bs + h * D;
    const __nv_bfloat16* dob = static_cast<const __nv_bfloat16*>(a.d_o) + b * a.do_bs + h * D;
    const float* lse = a.lse + (static_cast<long long>(b) * a.Hq + h) * a.Sq;
    const float* del = a.delta + (static_cast<long long>(b) * a.Hq + h) * a.Sq;
    for (int ib = ib0; ib < ib1; ++ib) {
      __syncthreads();  // previous iteration's readers are done with sQ/sdO
      load_tile<D, THREADS>(sQ, qb, a.q_ts, ib * BQ, a.Sq);
      load_tile<D, THREADS>(sdO, dob, a.do_ts, ib * BQ, a.Sq);
      cp_commit();
      if (threadIdx.x < 64) {
        int i = ib * BQ + threadIdx.x;
        sLse[threadIdx.x] = i < a.Sq ? lse[i] * LOG2E : INFINITY;
        sDel[threadIdx.x] = i < a.Sq ? del[i] : 0.f;
      }
      cp_wait<0>();
      __syncthreads();

      float st[8][4], dpt[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f;
        dpt[i][0] = dpt[i][1] = dpt[i][2] = dpt[i][3] = 0.f;
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t ak[4], av[4];
        load_a<D>(sK, k0, kk, ak);
        load_a<D>(sV, k0, kk, av);
#pragma unroll
        for (int np = 0; np < 4; ++np) {
          uint32_t bq[4], bd[4];
          load_b_nk<D>(sQ, np * 16, kk, bq);
          load_b_nk<D>(sdO, np * 16, kk, bd);
          mma16816(st[2 * np], ak, bq[0], bq[1]);
          mma16816(st[2 * np + 1], ak, bq[2], bq[3]);
          mma16816(dpt[2 * np], av, bd[0], bd[1]);
          mma16816(dpt[2 * np + 1], av, bd[2], bd[3]);
        }
      }
      uint32_t pf[4][4], dsf[4][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        float p[4], ds[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int il = nt * 8 + 2 * t + (e & 1);
          int i = ib * BQ + il;
          int key = (e < 2) ? key0 : key1;
          bool ok = i < a.Sq && allowed(a.q_offset + i, key, a.Sk, a.causal, a.window);
          p[e] = ok ? exp2f(st[nt][e] * c - sLse[il]) : 0.f;
          ds[e] = p[e] * (dpt[nt][e] - sDel[il]);
        }
        pf[nt >> 1][(nt & 1) * 2] = pack_bf16(p[0], p[1]);
        pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
        dsf[nt >> 1][(nt & 1) * 2] = pack_bf16(ds[0], ds[1]);
        dsf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(ds[2], ds[3]);
      }
#pragma unroll
      for (int k2 = 0; k2 < 4; ++k2) {
#pragma unroll
        for (int dp = 0; dp < DW / 16; ++dp) {
          uint32_t bo[4], bq[4];
          load_b_kn<D>(sdO, k2 * 16, d0 + dp * 16, bo);
          load_b_kn<D>(sQ, k2 * 16, d0 + dp * 16, bq);
          mma16816(dv[2 * dp], pf[k2], bo[0], bo[1]);
          mma16816(dv[2 * dp + 1], pf[k2], bo[2], bo[3]);
          mma16816(dk[2 * dp], dsf[k2], bq[0], bq[1]);
          mma16816(dk[2 * dp + 1], dsf[k2], bq[2], bq[3]);
        }
      }
    }
  }
  cp_wait<0>();
  __nv_bfloat16* dkb = static_cast<__nv_bfloat16*>(a.dk) + b * a.dk_bs + hk * D + d0;
  __nv_bfloat16* dvb = static_cast<__nv_bfloat16*>(a.dv) + b * a.dv_bs + hk * D + d0;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    int key = n0 + k0 + g + r * 8;
    if (key >= a.Sk) continue;
#pragma unroll
    for (int i = 0; i < DW / 8; ++i) {
      *reinterpret_cast<uint32_t*>(dkb + static_cast<long long>(key) * a.dk_ts + i * 8 + 2 * t) =
          pack_bf16(dk[i][2 * r] * a.scale, dk[i][2 * r + 1] * a.scale);
      *reinterpret_cast<uint32_t*>(dvb + static_cast<long long>(key) * a.dv_ts + i * 8 + 2 * t) =
          pack_bf16(dv[i][2 * r], dv[i][2 * r + 1]);
    }
  }
}

// dQ: CTA owns 64 query rows of one head and sweeps the key blocks they can see.
template <int D>
__global__ void __launch_bounds__(128) flash_bwd_dq_kernel(FlashArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int TILE = 64 * D * 2;
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + TILE;
  uint8_t* sK = smem + 2 * TILE;
  uint8_t* sV = smem + 3 * TILE;
  const int m0 = blockIdx.x * BQ, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const __nv_bfloat16* qb = static_cast<const __nv_bfloat16*>(a.q) + b * a.q_bs + h * D;
  const __nv_bfloat16* dob = static_cast<const __nv_bfloat16*>(a.d_o) + b * a.do_bs + h * D;
  const __nv_bfloat16* kb = static_cast<const __nv_bfloat16*>(a.k) + b * a.k_bs + hk * D;
  const __nv_bfloat16* vb = static_cast<const __nv_bfloat16*>(a.v) + b * a.v_bs + hk * D;
  load_tile<D, 128>(sQ, qb, a.q_ts, m0, a.Sq);
  load_tile<D, 128>(sdO, dob, a.do_ts, m0, a.Sq);
  cp_commit();
  const int r0 = warp * 16;
  const int row0 = m0 + r0 + g, row1 = row0 + 8;
  const float* lse = a.lse + (static_cast<long long>(b) * a.Hq + h) * a.Sq;
  const float* del = a.delta + (static_cast<long long>(b) * a.Hq + h) * a.Sq;
  const float lse0 = row0 < a.Sq ? lse[row0] * LOG2E : INFINITY, lse1 = row1 < a.Sq ? lse[row1] * LOG2E : INFINITY;
  const float del0 = row0 < a.Sq ? del[row0] : 0.f, del1 = row1 < a.Sq ? del[row1] : 0.f;
  const float c = a.scale * LOG2E;
  float dq[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;

  int j_hi = a.causal ? min(a.Sk, a.q_offset + m0 + BQ) : a.Sk;
  int j_lo = a.window > 0 ? max(0, a.q_offset + m0 - a.window + 1) : 0;
  const int jb0 = j_lo / BKV, jb1 = (j_hi + BKV - 1) / BKV;
  for (int jb = jb0; jb < jb1; ++jb) {
    __syncthreads();
    load_tile<D, 128>(sK, kb, a.k_ts, jb * BKV, a.Sk);
    load_tile<D, 128>(sV, vb, a.v_ts, jb * BKV, a.Sk);
    cp_commit();
    cp_wait<0>();
    __syncthreads();
    float s[8][4], dp[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
    }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t aq[4], ad[4];
      load_a<D>(sQ, r0, kk, aq);
      load_a<D>(sdO, r0, kk, ad);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bk[4], bv[4];
        load_b_nk<D>(sK, np * 16, kk, bk);
        load_b_nk<D>(sV, np * 16, kk, bv);
        mma16816(s[2 * np], aq, bk[0], bk[1]);
        mma16816(s[2 * np + 1], aq, bk[2], bk[3]);
        mma16816(dp[2 * np], ad, bv[0], bv[1]);
        mma16816(dp[2 * np + 1], ad, bv[2], bv[3]);
      }
    }
    uint32_t dsf[4][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      float ds[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int j = jb * BKV + nt * 8 + 2 * t + (e & 1);
        int row = (e < 2) ? row0 : row1;
        bool ok = row < a.Sq && allowed(a.q_offset + row, j, a.Sk, a.causal, a.window);
        float p = ok ? exp2f(s[nt][e] * c - ((e < 2) ? lse0 : lse1)) : 0.f;
        ds[e] = p * (dp[nt][e] - ((e < 2) ? del0 : del1));
      }
      dsf[nt >> 1][(nt & 1) * 2] = pack_bf16(ds[0], ds[1]);
      dsf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(ds[2], ds[3]);
    }
#pragma unroll
    for (int k2 = 0; k2 < 4; ++k2) {
#pragma unroll
      for (int dd = 0; dd < D / 16; ++dd) {
        uint32_t bk[4];
        load_b_kn<D>(sK, k2 * 16, dd * 16, bk);
        mma16816(dq[2 * dd], dsf[k2], bk[0], bk[1]);
        mma16816(dq[2 * dd + 1], dsf[k2], bk[2], bk[3]);
      }
    }
  }
  cp_wait<0>();
  __nv_bfloat16* dqb = static_cast<__nv_bfloat16*>(a.dq) + b * a.dq_bs + h * D;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    int row = r ? row1 : row0;
    if (row >= a.Sq) continue;
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
      *reinterpret_cast<uint32_t*>(dqb + static_cast<long long>(row) * a.dq_ts + i * 8 + 2 * t) =
          pack_bf16(dq[i][2 * r] * a.scale, dq[i][2 * r + 1] * a.scale);
  }
}

template <typename K>
const char* set_smem(K kern, size_t bytes) {
  if (bytes > 48 * 1024 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)) != cudaSuccess)
    return "flash: cudaFuncSetAttribute failed";
  return nullptr;
}

template <int D>
const char* fwd_d(const FlashArgs& a, cudaStream_t s) {
  size_t smem = 5 * 64 * D * 2;
  if (const char* e = set_smem(flash_fwd_kernel<D>, smem)) return e;
  dim3 grid((a.Sq + BQ - 1) / BQ, a.Hq, a.B);
  flash_fwd_kernel<D><<<grid, 128, smem, s>>>(a);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "flash_fwd launch failed";
}

template <int D, int DSPLIT>
const char* bwd_d(const FlashArgs& a, cudaStream_t s) {
  long long warps = static_cast<long long>(a.B) * a.Sq * a.Hq;
  flash_delta_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, s>>>(a);
  count_launch();
  size_t smem = 4 * 64 * D * 2 + 512;
  if (const char* e = set_smem(flash_bwd_dkv_kernel<D, DSPLIT>, smem)) return e;
  dim3 gkv((a.Sk + BKV - 1) / BKV, a.Hkv, a.B);
  flash_bwd_dkv_kernel<D, DSPLIT><<<gkv, 128 * DSPLIT, smem, s>>>(a);
  count_launch();
  size_t smem2 = 4 * 64 * D * 2;
  if (const char* e = set_smem(flash_bwd_dq_kernel<D>, smem2)) return e;
  dim3 gq((a.Sq + BQ - 1) / BQ, a.Hq, a.B);
  flash_bwd_dq_kernel<D><<<gq, 128, smem2, s>>>(a);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "flash_bwd launch failed";
}

const char* check(const FlashArgs& a) {
  if (a.Hq % a.Hkv) return "flash: Hq must be a multiple of Hkv";
  if ((a.q_ts % 8) || (a.k_ts % 8) || (a.v_ts % 8) || (a.q_bs % 8) || (a.k_bs % 8) || (a.v_bs % 8))
    return "flash: strides must be multiples of 8 elements (16-byte rows)";
  if ((reinterpret_cast<uintptr_t>(a.q) & 15) || (reinterpret_cast<uintptr_t>(a.k) & 15) ||
      (reinterpret_cast<uintptr_t>(a.v) & 15))
    return "flash: base pointers must be 16-byte aligned";
  return nullptr;
}

}  // namespace

const char* flash_fwd(const FlashArgs& a, cudaStream_t s) {
  if (a.B == 0 || a.Sq == 0) return nullptr;
  if (const char* e = check(a)) return e;
  switch (a.D) {
    case 64: return fwd_d<64>(a, s);
    case 128: return fwd_d<128>(a, s);
    case 256: return fwd_d<256>(a, s);
    default: return "flash: head_dim must be 64, 128 or 256";
  }
}

const char* flash_bwd(const FlashArgs& a, cudaStream_t s) {
  if (a.B == 0 || a.Sq == 0) return nullptr;
  if (const char* e = check(a)) return e;
  switch (a.D) {
    case 64: return bwd_d<64, 1>(a, s);
    case 128: return bwd_d<128, 1>(a, s);
    case 256: return bwd_d<256, 2>(a, s);
    default: return "flash: head_dim must be 64, 128 or 256";
  }
}

}  // namespace ferrl
