// Causal flash-attention forward on the 5th-generation tensor cores (head_dim 128 or 256, optional sliding window).
//
// One CTA owns 128 query rows of one head and walks the key/value sequence in tiles of 128 keys:
//
//   warp 0      TMA producer: Q once, then K tiles [128 keys x 128 dims] and V^T tiles
//               [128 dims x 128 keys] into two-deep rings (128B swizzle, no cluster multicast)
//   warp 1      one thread issues tcgen05.mma: S = Q K^T into a double-buffered TMEM accumulator
//               (tile j+1's scores are computed while tile j's softmax runs), then O_j = P V
//   warps 2-5   softmax: each thread owns one query row, reads its scores with tcgen05.ld (row max
//               and row sum need no shuffles), writes P as bf16 into shared memory in the swizzled
//               K-major layout the MMA reads, rescales its fp32 output row while the P V MMA runs,
//               and adds the tile's P V from TMEM
//
// V is transposed once per call by a small kernel so that both MMAs read K-major operands written
// by TMA.  The warp-level kernel in flash_attn.cu (mma.sync) reaches ~13 % of the measured bf16
// peak on these shapes; it stays as the path for other head dims and query offsets, and its
// backward consumes the log-sum-exp this kernel writes.  Head_dim 256 and sliding windows take the third
// form at the end of this file.  Reference: candle's flash-attn binding /
// eager GQA attention (crates/ferrl/src/dense.rs attention path).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"
#include "../gemm/tc_common.cuh"

namespace ferrl {
namespace {

using namespace tc;

constexpr int FD = 128;                 // head dim
constexpr int FT = 128;                 // query rows per CTA and keys per tile
constexpr int ATOM = FT * 64 * 2;       // one [128 rows x 64 cols] swizzle atom: 16 KB
constexpr int TILE = 2 * ATOM;          // [128 x 128] bf16 tile: 32 KB
constexpr float kLog2e = 1.4426950408889634f;

struct FlashTcParams {
  __nv_bfloat16* out; long long o_bs, o_ts;
  float* lse;                           // [B, Hq, S] or null
  int B, S, Hq, Hkv;
  float scale;
  int* status;
};

// vt[(b, hk, d), s] = v[b, s, hk, d]; zero for s in [S, S_pad)
__global__ void transpose_v_kernel(const __nv_bfloat16* __restrict__ v, long long v_bs, long long v_ts,
                                   __nv_bfloat16* __restrict__ vt, int S, int S_pad, int Hkv) {
  __shared__ __nv_bfloat16 tile[64][FD + 2];
  const int s0 = blockIdx.x * 64, hk = blockIdx.y, b = blockIdx.z;
  for (int i = threadIdx.x; i < 64 * (FD / 2); i += blockDim.x) {
    const int r = i / (FD / 2), c2 = i % (FD / 2);
    __nv_bfloat162 val = __floats2bfloat162_rn(0.f, 0.f);
    if (s0 + r < S) val = *reinterpret_cast<const __nv_bfloat162*>(v + b * v_bs + static_cast<long long>(s0 + r) * v_ts + hk * FD + 2 * c2);
    tile[r][2 * c2] = val.x;
    tile[r][2 * c2 + 1] = val.y;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < FD * 32; i += blockDim.x) {
    const int d = i / 32, r2 = i % 32;
    __nv_bfloat162 val;
    val.x = tile[2 * r2][d];
    val.y = tile[2 * r2 + 1][d];
    *reinterpret_cast<__nv_bfloat162*>(vt + (static_cast<long long>(b) * Hkv + hk) * FD * S_pad + static_cast<long long>(d) * S_pad + s0 + 2 * r2) = val;
  }
}

__global__ void __launch_bounds__(192, 1)
flash_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmVt, FlashTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                    // 32 KB
  uint8_t* sK = sQ + TILE;               // 2 x 32 KB
  uint8_t* sV = sK + 2 * TILE;           // 2 x 32 KB
  uint8_t* sP = sV + 2 * TILE;           // 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + TILE);
  uint64_t* q_full = bars;               // [1]
  uint64_t* k_full = bars + 1;           // [2]
  uint64_t* k_empty = bars + 3;          // [2]
  uint64_t* v_full = bars + 5;           // [2]
  uint64_t* v_empty = bars + 7;          // [2]
  uint64_t* s_full = bars + 9;           // [2]
  uint64_t* s_empty = bars + 11;         // [2]
  uint64_t* p_full = bars + 13;          // [1]
  uint64_t* pv_full = bars + 14;         // [1]
  uint64_t* pv_empty = bars + 15;        // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.S + FT - 1) / FT;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);     // longest rows first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int hk = hq / (p.Hq / p.Hkv);
  const int q0 = qt * FT;
  const int n_kv = qt + 1;                                    // causal: tiles 0..qt

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_full, 1);
    mbar_init(pv_empty, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS0 = tmem_base, tS1 = tmem_base + 128;
  const uint32_t tPV = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      mbar_expect_tx(q_full, TILE);
      tma_load_2d(sQ, &tmQ, q_full, hq * FD, b * p.S + q0);
      tma_load_2d(sQ + ATOM, &tmQ, q_full, hq * FD + 64, b * p.S + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_expect_tx(&k_full[st], TILE);
        tma_load_2d(sK + st * TILE, &tmK, &k_full[st], hk * FD, b * p.S + j * FT);
        tma_load_2d(sK + st * TILE + ATOM, &tmK, &k_full[st], hk * FD + 64, b * p.S + j * FT);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_expect_tx(&v_full[st], TILE);
        tma_load_2d(sV + st * TILE, &tmVt, &v_full[st], j * FT, (b * p.Hkv + hk) * FD);
        tma_load_2d(sV + st * TILE + ATOM, &tmVt, &v_full[st], j * FT + 64, (b * p.Hkv + hk) * FD);
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(10000);   // let copies in flight land before shared memory goes away
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = make_idesc_bf16(128, 128);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
        tc_fence_after();
        const uint64_t dq = make_smem_desc(smem_u32(sQ)), dk = make_smem_desc(smem_u32(sK + st * TILE));
        const uint32_t ts = st ? tS1 : tS0;
#pragma unroll
        for (int ks = 0; ks < FD / 16; ++ks) {
          const uint32_t off = (ks >> 2) * ATOM + (ks & 3) * 32;
          umma(ts, desc_adv(dq, off), desc_adv(dk, off), idesc, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kStatusWaitTimeoutMma);
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) ok = issue_qk(j + 1);
        if (!ok) break;
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(p_full, j & 1, abort_flag, p.status, kStatusWaitTimeoutMma) ||
            !mbar_wait(&v_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutMma) ||
            !mbar_wait(pv_empty, (j & 1) ^ 1, abort_flag, p.status, kStatusWaitTimeoutMma)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t dp = make_smem_desc(smem_u32(sP)), dvt = make_smem_desc(smem_u32(sV + st * TILE));
#pragma unroll
        for (int ks = 0; ks < FT / 16; ++ks) {
          const uint32_t off = (ks >> 2) * ATOM;
          umma(tPV, desc_adv(dp, off + (ks & 3) * 32), desc_adv(dvt, off + (ks & 3) * 32), idesc, ks > 0 ? 1u : 0u);
        }
        umma_commit(pv_full);
        umma_commit(&v_empty[st]);
      }
    }
  } else {
    // -------------------------------------------------------------------- softmax + output (one row per thread)
    const int q = warp & 3;
    const int r = q * 32 + lane;                  // row inside the tile == TMEM lane
    const int row = q0 + r;                       // query position
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const float c = p.scale * kLog2e;
    float m_run = -INFINITY, l_run = 0.f;
    float o[FD];
#pragma unroll
    for (int i = 0; i < FD; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * FT;
      const int limit = min(p.S, (j == qt) ? row + 1 : p.S) - k0;     // keys [0, limit) of this tile are visible
      // pass 1: row maximum
      float mx = m_run;
#pragma unroll 1
      for (int cc = 0; cc < FT; cc += 32) {
        uint32_t v[32];
        tmem_ld32((st ? tS1 : tS0) + lane_sel + cc, v);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (cc + e < limit) mx = fmaxf(mx, __uint_as_float(v[e]));
      }
      const float corr = (m_run == -INFINITY) ? 0.f : exp2f((m_run - mx) * c);
      const float mc = (mx == -INFINITY) ? 0.f : mx * c;
      // pass 2: probabilities -> bf16 -> swizzled K-major tile; row sum
      float ps = 0.f;
#pragma unroll 1
      for (int cc = 0; cc < FT; cc += 32) {
        uint32_t v[32];
        tmem_ld32((st ? tS1 : tS0) + lane_sel + cc, v);
        tmem_ld_wait();
        float pr[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          pr[e] = (cc + e < limit) ? exp2f(__uint_as_float(v[e]) * c - mc) : 0.f;
          ps += pr[e];
        }
        uint8_t* dst = sP + (cc >> 6) * ATOM + r * 128;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint4 w;
          __nv_bfloat162* wh = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
          for (int e = 0; e < 4; ++e) wh[e] = __floats2bfloat162_rn(pr[ch * 8 + 2 * e], pr[ch * 8 + 2 * e + 1]);
          const int chunk = ((cc & 63) >> 3) + ch;
          *reinterpret_cast<uint4*>(dst + ((chunk ^ (r & 7)) << 4)) = w;
        }
      }
      // scores of this buffer are consumed; P is written
      tc_fence_before();
      fence_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[st]);
        mbar_arrive(p_full);
      }
      l_run = l_run * corr + ps;
      m_run = mx;
      // rescale the running output while the tensor cores compute P V
#pragma unroll
      for (int i = 0; i < FD; ++i) o[i] *= corr;
      if (!mbar_wait(pv_full, j & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int cc = 0; cc < FD; cc += 32) {
        uint32_t v[32];
        tmem_ld32(tPV + lane_sel + cc, v);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[cc + e] += __uint_as_float(v[e]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pv_empty);
    }
    if (ok && row < p.S) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.out + b * p.o_bs + static_cast<long long>(row) * p.o_ts + hq * FD;
#pragma unroll
      for (int ch = 0; ch < FD / 8; ++ch) {
        uint4 w;
        __nv_bfloat162* wh = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
        for (int e = 0; e < 4; ++e) wh[e] = __floats2bfloat162_rn(o[ch * 8 + 2 * e] * inv, o[ch * 8 + 2 * e + 1] * inv);
        reinterpret_cast<uint4*>(orow)[ch] = w;
      }
      if (p.lse)
        p.lse[(static_cast<long long>(b) * p.Hq + hq) * p.S + row] = (l_run > 0.f) ? m_run * p.scale + logf(l_run) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// Second form of the same kernel: the running output stays in TMEM (the P V MMAs accumulate into it
// across tiles), a thread reads its score row once and keeps it in registers, P is double-buffered
// and the output is rescaled lazily - only when the row maximum grew by more than 2^8 since the last
// rescale.  Per tile a softmax thread then has one round of TMEM loads instead of three.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// tcgen05.mma with the A operand in tensor memory (row i in lane i, two bf16 per 32-bit column)
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accum)
      : "memory");
}

// PT: P stays in tensor memory (written with tcgen05.st as packed bf16, read by the P V MMAs as their
// A operand), so it costs neither shared-memory writes nor shared-memory read bandwidth.
template <bool PT>
__global__ void __launch_bounds__(192, 1)
flash_fwd_tc2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmVt, FlashTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                    // 32 KB
  uint8_t* sK = sQ + TILE;               // 2 x 32 KB
  uint8_t* sV = sK + 2 * TILE;           // 2 x 32 KB
  uint8_t* sP = sV + 2 * TILE;           // 2 x 32 KB (absent when P stays in tensor memory)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + (PT ? 0 : 2 * TILE));
  uint64_t* q_full = bars;               // [1]
  uint64_t* k_full = bars + 1;           // [2]
  uint64_t* k_empty = bars + 3;          // [2]
  uint64_t* v_full = bars + 5;           // [2]
  uint64_t* v_empty = bars + 7;          // [2]
  uint64_t* s_full = bars + 9;           // [2]
  uint64_t* s_empty = bars + 11;         // [2]
  uint64_t* p_full = bars + 13;          // [2] softmax wrote P[buf]
  uint64_t* p_free = bars + 15;          // [2] the P V MMAs reading P[buf] have retired (O includes that tile)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.S + FT - 1) / FT;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);     // longest rows first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int hk = hq / (p.Hq / p.Hkv);
  const int q0 = qt * FT;
  const int n_kv = qt + 1;                                    // causal: tiles 0..qt

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&p_full[i], 4);
      mbar_init(&p_free[i], 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS0 = tmem_base, tS1 = tmem_base + 128;
  const uint32_t tO = tmem_base + 256;     // running output, accumulated by the P V MMAs across tiles
  const uint32_t tP0 = tmem_base + 384;    // PT: two P buffers of 64 columns (128 keys as bf16 pairs)

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      mbar_expect_tx(q_full, TILE);
      tma_load_2d(sQ, &tmQ, q_full, hq * FD, b * p.S + q0);
      tma_load_2d(sQ + ATOM, &tmQ, q_full, hq * FD + 64, b * p.S + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_expect_tx(&k_full[st], TILE);
        tma_load_2d(sK + st * TILE, &tmK, &k_full[st], hk * FD, b * p.S + j * FT);
        tma_load_2d(sK + st * TILE + ATOM, &tmK, &k_full[st], hk * FD + 64, b * p.S + j * FT);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_expect_tx(&v_full[st], TILE);
        tma_load_2d(sV + st * TILE, &tmVt, &v_full[st], j * FT, (b * p.Hkv + hk) * FD);
        tma_load_2d(sV + st * TILE + ATOM, &tmVt, &v_full[st], j * FT + 64, (b * p.Hkv + hk) * FD);
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(10000);   // let copies in flight land before shared memory goes away
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA warp: all lanes walk the loop, one issues
    constexpr uint32_t idesc = make_idesc_bf16(128, 128);
    const uint64_t dq = make_smem_desc(smem_u32(sQ));
    auto issue_qk = [&](int j) -> bool {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait_warp(&k_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
      if (!mbar_wait_warp(&s_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
      tc_fence_after();
      const uint64_t dk = make_smem_desc(smem_u32(sK + st * TILE));
      const uint32_t ts = st ? tS1 : tS0;
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < FD / 16; ++ks) {
          const uint32_t off = (ks >> 2) * ATOM + (ks & 3) * 32;
          umma(ts, desc_adv(dq, off), desc_adv(dk, off), idesc, ks > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
      }
      __syncwarp();
      return true;
    };
    bool ok = mbar_wait_warp(q_full, 0, abort_flag, p.status, kStatusWaitTimeoutMma);
    if (ok) ok = issue_qk(0);
    for (int j = 0; j < n_kv && ok; ++j) {
      if (j + 1 < n_kv) ok = issue_qk(j + 1);
      if (!ok) break;
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const int pb = j & 1;
      if (!mbar_wait_warp(&p_full[pb], ph, abort_flag, p.status, kStatusWaitTimeoutMma) ||
          !mbar_wait_warp(&v_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutMma)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint64_t dp = make_smem_desc(smem_u32(sP + pb * TILE)), dvt = make_smem_desc(smem_u32(sV + st * TILE));
      const uint32_t acc0 = j > 0 ? 1u : 0u;
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < FT / 16; ++ks) {
          const uint32_t off = (ks >> 2) * ATOM + (ks & 3) * 32;
          if (PT) umma_ts(tO, tP0 + pb * 64 + ks * 8, desc_adv(dvt, off), idesc, ks > 0 ? 1u : acc0);
          else umma(tO, desc_adv(dp, off), desc_adv(dvt, off), idesc, ks > 0 ? 1u : acc0);
        }
        umma_commit(&p_free[pb]);
        umma_commit(&v_empty[st]);
      }
      __syncwarp();
    }
  } else {
    // -------------------------------------------------------------------- softmax + output (one row per thread)
    const int q = warp & 3;
    const int r = q * 32 + lane;                  // row inside the tile == TMEM lane
    const int row = q0 + r;                       // query position
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const float c = p.scale * kLog2e;
    float m_used = -INFINITY, l_run = 0.f;      // probabilities are taken relative to m_used
    const bool rows_ok = __all_sync(0xffffffffu, row < p.S);
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait_warp(&s_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      // the whole score row in registers: one round of TMEM loads, one wait
      uint32_t sv[FT];
      tmem_ld32((st ? tS1 : tS0) + lane_sel + 0, sv + 0);
      tmem_ld32((st ? tS1 : tS0) + lane_sel + 32, sv + 32);
      tmem_ld32((st ? tS1 : tS0) + lane_sel + 64, sv + 64);
      tmem_ld32((st ? tS1 : tS0) + lane_sel + 96, sv + 96);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[st]);       // the next-but-one Q K^T may overwrite this buffer
      const int k0 = j * FT;
      const int limit = min(p.S, (j == qt) ? row + 1 : p.S) - k0;
      // tiles strictly below the diagonal need no mask (warp-uniform test); four independent chains
      // for the maximum and for the sum, a single warp per scheduler has no other way to hide latency
      const bool full = (j < qt) && rows_ok;
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (full) {
#pragma unroll
        for (int e = 0; e < FT; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sv[e]));
      } else {
#pragma unroll
        for (int e = 0; e < FT; ++e)
          if (e < limit) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sv[e]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_used, mx);
      // Lazy rescale: O (in TMEM) and l are only brought to the new maximum when it grew by more than
      // 2^8 since the last rescale; smaller growth just makes the probabilities of this tile larger.
      const bool need = (j > 0) && ((m_new - m_used) * c > 8.f);
      if (j == 0) m_used = m_new;
      if (__any_sync(0xffffffffu, need)) {
        // O must contain every earlier tile before it is touched: wait for P V of tile j-1
        if (!mbar_wait_warp(&p_free[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
        tc_fence_after();
        const float corr = need ? exp2f((m_used - m_new) * c) : 1.f;
        if (need) {
          m_used = m_new;
          l_run *= corr;
        }
#pragma unroll 1
        for (int cc = 0; cc < FD; cc += 32) {
          uint32_t ov[32];
          tmem_ld32(tO + lane_sel + cc, ov);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * corr);
          tmem_st32(tO + lane_sel + cc, ov);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      // P[j & 1] is free again once P V of tile j-2 has retired
      const int pb = j & 1;
      if (j >= 2 && !mbar_wait_warp(&p_free[pb], ((j >> 1) - 1) & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      const float mc = m_used * c;
      float ps = 0.f;
      if (PT) {
        // packed in place: word i0/2 replaces a score that has already been consumed
        float ps4[4] = {0.f, 0.f, 0.f, 0.f};
        if (full) {
#pragma unroll
          for (int i0 = 0; i0 < FT; i0 += 2) {
            const float p0 = exp2f(__uint_as_float(sv[i0]) * c - mc);
            const float p1 = exp2f(__uint_as_float(sv[i0 + 1]) * c - mc);
            ps4[(i0 >> 1) & 3] += p0 + p1;
            __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            sv[i0 >> 1] = *reinterpret_cast<uint32_t*>(&h);
          }
        } else {
#pragma unroll
          for (int i0 = 0; i0 < FT; i0 += 2) {
            const float p0 = (i0 < limit) ? exp2f(__uint_as_float(sv[i0]) * c - mc) : 0.f;
            const float p1 = (i0 + 1 < limit) ? exp2f(__uint_as_float(sv[i0 + 1]) * c - mc) : 0.f;
            ps4[(i0 >> 1) & 3] += p0 + p1;
            __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            sv[i0 >> 1] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        ps = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
        l_run += ps;
        tmem_st32(tP0 + pb * 64 + lane_sel, sv);
        tmem_st32(tP0 + pb * 64 + lane_sel + 32, sv + 32);
        tmem_st_wait();
        tc_fence_before();
      } else {
        uint8_t* prow = sP + pb * TILE + r * 128;
        float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ch = 0; ch < FT / 8; ++ch) {
          uint4 w;
          __nv_bfloat162* wh = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i0 = ch * 8 + 2 * e;
            const float p0 = (full || i0 < limit) ? exp2f(__uint_as_float(sv[i0]) * c - mc) : 0.f;
            const float p1 = (full || i0 + 1 < limit) ? exp2f(__uint_as_float(sv[i0 + 1]) * c - mc) : 0.f;
            ps4[e] += p0 + p1;
            wh[e] = __floats2bfloat162_rn(p0, p1);
          }
          *reinterpret_cast<uint4*>(prow + (ch >> 3) * ATOM + (((ch & 7) ^ (r & 7)) << 4)) = w;
        }
        ps = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
        l_run += ps;
        fence_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[pb]);
    }
    // the last P V completes the output
    if (ok && n_kv > 0 &&
        !mbar_wait_warp(&p_free[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue))
      ok = false;
    tc_fence_after();
    if (ok) {      // warp-uniform: the TMEM loads are warp-collective, only the stores are per row
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.out + b * p.o_bs + static_cast<long long>(row) * p.o_ts + hq * FD;
#pragma unroll 1
      for (int cc = 0; cc < FD; cc += 32) {
        uint32_t ov[32];
        __syncwarp();   // lanes that skipped the stores rejoin before the collective load
        tmem_ld32(tO + lane_sel + cc, ov);
        tmem_ld_wait();
        if (row < p.S) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 w;
            __nv_bfloat162* wh = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              wh[e] = __floats2bfloat162_rn(__uint_as_float(ov[ch * 8 + 2 * e]) * inv, __uint_as_float(ov[ch * 8 + 2 * e + 1]) * inv);
            reinterpret_cast<uint4*>(orow + cc)[ch] = w;
          }
        }
      }
      if (p.lse && row < p.S)
        p.lse[(static_cast<long long>(b) * p.Hq + hq) * p.S + row] = (l_run > 0.f) ? m_used * p.scale + logf(l_run) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}


// Third form, generalised from the second (output and P in tensor memory): head_dim HD of 128 or 256 and an
// optional sliding window.  A CTA still owns 128 query rows; keys come in tiles of KT (128 for head_dim 128,
// 64 for head_dim 256, so that Q, two K tiles and two V^T tiles fit in shared memory and S x2, O and P x2 fit
// in the 512 TMEM columns: 3 KT + HD).  With a window of w keys, query i sees keys (i - w, i]: the walk starts
// at the first tile any row of the CTA can see, and only the tiles that cut the window's lower edge or the
// diagonal pay for a mask.  A row may see nothing in the CTA's first tiles; its running maximum then stays at
// -inf, its probabilities are zero, and the first visible tile rescales the (zero) output by zero.
template <int HD>
__global__ void transpose_v_hd_kernel(const __nv_bfloat16* __restrict__ v, long long v_bs, long long v_ts,
                                      __nv_bfloat16* __restrict__ vt, int S, int S_pad, int Hkv) {
  extern __shared__ __nv_bfloat16 tv_tile[];          // [64][HD + 2]
  const int s0 = blockIdx.x * 64, hk = blockIdx.y, b = blockIdx.z;
  for (int i = threadIdx.x; i < 64 * (HD / 2); i += blockDim.x) {
    const int r = i / (HD / 2), c2 = i % (HD / 2);
    __nv_bfloat162 val = __floats2bfloat162_rn(0.f, 0.f);
    if (s0 + r < S) val = *reinterpret_cast<const __nv_bfloat162*>(v + b * v_bs + static_cast<long long>(s0 + r) * v_ts + hk * HD + 2 * c2);
    tv_tile[r * (HD + 2) + 2 * c2] = val.x;
    tv_tile[r * (HD + 2) + 2 * c2 + 1] = val.y;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < HD * 32; i += blockDim.x) {
    const int d = i / 32, r2 = i % 32;
    __nv_bfloat162 val;
    val.x = tv_tile[(2 * r2) * (HD + 2) + d];
    val.y = tv_tile[(2 * r2 + 1) * (HD + 2) + d];
    *reinterpret_cast<__nv_bfloat162*>(vt + (static_cast<long long>(b) * Hkv + hk) * HD * S_pad + static_cast<long long>(d) * S_pad + s0 + 2 * r2) = val;
  }
}

template <int HD, int KT>
struct Tc3Cfg {
  static constexpr int Q_BYTES = FT * HD * 2;          // HD/64 atoms of [128 rows x 64 cols]
  static constexpr int K_ATOM = KT * 128;              // [KT keys x 64 dims]
  static constexpr int K_BYTES = (HD / 64) * K_ATOM;
  static constexpr int V_ATOM = HD * 128;              // [HD dims x 64 keys]
  static constexpr int V_BYTES = (KT / 64) * V_ATOM;
  static constexpr int SMEM = Q_BYTES + 2 * K_BYTES + 2 * V_BYTES + 1024 + 256;
  static_assert(3 * KT + HD <= 512, "tensor memory columns");
};

template <int HD, int KT>
__global__ void __launch_bounds__(192, 1)
flash_fwd_tc3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmVt, FlashTcParams p, int window) {
  using C = Tc3Cfg<HD, KT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::Q_BYTES;
  uint8_t* sV = sK + 2 * C::K_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * C::V_BYTES);
  uint64_t* q_full = bars;               // [1]
  uint64_t* k_full = bars + 1;           // [2]
  uint64_t* k_empty = bars + 3;          // [2]
  uint64_t* v_full = bars + 5;           // [2]
  uint64_t* v_empty = bars + 7;          // [2]
  uint64_t* s_full = bars + 9;           // [2]
  uint64_t* s_empty = bars + 11;         // [2]
  uint64_t* p_full = bars + 13;          // [2]
  uint64_t* p_free = bars + 15;          // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.S + FT - 1) / FT;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);     // longest rows first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int hk = hq / (p.Hq / p.Hkv);
  const int q0 = qt * FT;
  const int last_row = min(q0 + FT, p.S) - 1;
  const int j_lo = window > 0 ? max(0, q0 - window + 1) / KT : 0;
  const int n_kv = last_row / KT - j_lo + 1;                   // key tiles j_lo .. last_row / KT

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
      mbar_init(&p_full[i], 4);
      mbar_init(&p_free[i], 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS0 = tmem_base, tS1 = tmem_base + KT;
  const uint32_t tO = tmem_base + 2 * KT;          // running output [128 x HD]
  const uint32_t tP0 = tO + HD;                    // two P buffers of KT / 2 columns (KT keys as bf16 pairs)

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      mbar_expect_tx(q_full, C::Q_BYTES);
#pragma unroll
      for (int a = 0; a < HD / 64; ++a) tma_load_2d(sQ + a * ATOM, &tmQ, q_full, hq * HD + a * 64, b * p.S + q0);
      for (int jj = 0; jj < n_kv; ++jj) {
        const int j = j_lo + jj, st = jj & 1;
        const uint32_t ph = (jj >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_expect_tx(&k_full[st], C::K_BYTES);
#pragma unroll
        for (int a = 0; a < HD / 64; ++a)
          tma_load_2d(sK + st * C::K_BYTES + a * C::K_ATOM, &tmK, &k_full[st], hk * HD + a * 64, b * p.S + j * KT);
        if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_expect_tx(&v_full[st], C::V_BYTES);
#pragma unroll
        for (int a = 0; a < KT / 64; ++a)
          tma_load_2d(sV + st * C::V_BYTES + a * C::V_ATOM, &tmVt, &v_full[st], j * KT + a * 64, (b * p.Hkv + hk) * HD);
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(10000);   // let copies in flight land before shared memory goes away
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA warp: all lanes walk the loop, one issues
    constexpr uint32_t idesc_qk = make_idesc_bf16(128, KT), idesc_pv = make_idesc_bf16(128, HD);
    const uint64_t dq = make_smem_desc(smem_u32(sQ));
    auto issue_qk = [&](int jj) -> bool {
      const int st = jj & 1;
      const uint32_t ph = (jj >> 1) & 1;
      if (!mbar_wait_warp(&k_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
      if (!mbar_wait_warp(&s_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
      tc_fence_after();
      const uint64_t dk = make_smem_desc(smem_u32(sK + st * C::K_BYTES));
      const uint32_t ts = st ? tS1 : tS0;
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          umma(ts, desc_adv(dq, (ks >> 2) * ATOM + (ks & 3) * 32), desc_adv(dk, (ks >> 2) * C::K_ATOM + (ks & 3) * 32), idesc_qk,
               ks > 0 ? 1u : 0u);
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
      }
      __syncwarp();
      return true;
    };
    bool ok = mbar_wait_warp(q_full, 0, abort_flag, p.status, kStatusWaitTimeoutMma);
    if (ok) ok = issue_qk(0);
    for (int jj = 0; jj < n_kv && ok; ++jj) {
      if (jj + 1 < n_kv) ok = issue_qk(jj + 1);
      if (!ok) break;
      const int st = jj & 1;
      const uint32_t ph = (jj >> 1) & 1;
      if (!mbar_wait_warp(&p_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutMma) ||
          !mbar_wait_warp(&v_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutMma)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint64_t dvt = make_smem_desc(smem_u32(sV + st * C::V_BYTES));
      const uint32_t acc0 = jj > 0 ? 1u : 0u;
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < KT / 16; ++ks)
          umma_ts(tO, tP0 + st * (KT / 2) + ks * 8, desc_adv(dvt, (ks >> 2) * C::V_ATOM + (ks & 3) * 32), idesc_pv,
                  ks > 0 ? 1u : acc0);
        umma_commit(&p_free[st]);
        umma_commit(&v_empty[st]);
      }
      __syncwarp();
    }
  } else {
    // -------------------------------------------------------------------- softmax + output (one row per thread)
    const int q = warp & 3;
    const int r = q * 32 + lane;                  // row inside the tile == TMEM lane
    const int row = q0 + r;                       // query position
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const float c = p.scale * kLog2e;
    float m_used = -INFINITY, l_run = 0.f;      // probabilities are taken relative to m_used
    const bool rows_ok = __all_sync(0xffffffffu, row < p.S);
    bool ok = true;
    for (int jj = 0; jj < n_kv; ++jj) {
      const int j = j_lo + jj, st = jj & 1;
      const uint32_t ph = (jj >> 1) & 1;
      if (!mbar_wait_warp(&s_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[KT];
#pragma unroll
      for (int cc = 0; cc < KT; cc += 32) tmem_ld32((st ? tS1 : tS0) + lane_sel + cc, sv + cc);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[st]);       // the next-but-one Q K^T may overwrite this buffer
      const int k0 = j * KT;
      const int limit = min(p.S, row + 1) - k0;                       // keys [lo, limit) of this tile are visible
      const int lo = window > 0 ? row - window + 1 - k0 : -(1 << 30);
      // warp-uniform: no row of the CTA is cut by the diagonal, the window's lower edge or the sequence end
      const bool full = rows_ok && (k0 + KT - 1 <= q0) && (window == 0 || q0 + FT - window <= k0);
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (full) {
#pragma unroll
        for (int e = 0; e < KT; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sv[e]));
      } else {
#pragma unroll
        for (int e = 0; e < KT; ++e)
          if (e < limit && e >= lo) mx4[e & 3] = fmaxf(mx4[e & 3], __uint_as_float(sv[e]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_used, mx);
      // lazy rescale, as in the second form; a row that saw nothing so far (m_used = -inf) rescales by zero
      const bool need = (jj > 0) && (m_new > m_used) && ((m_new - m_used) * c > 8.f);
      if (jj == 0) m_used = m_new;
      if (__any_sync(0xffffffffu, need)) {
        if (!mbar_wait_warp(&p_free[(jj - 1) & 1], ((jj - 1) >> 1) & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
        tc_fence_after();
        const float corr = need ? ((m_used == -INFINITY) ? 0.f : exp2f((m_used - m_new) * c)) : 1.f;
        if (need) {
          m_used = m_new;
          l_run *= corr;
        }
#pragma unroll 1
        for (int cc = 0; cc < HD; cc += 32) {
          uint32_t ov[32];
          tmem_ld32(tO + lane_sel + cc, ov);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * corr);
          tmem_st32(tO + lane_sel + cc, ov);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      // P[jj & 1] is free again once P V of tile jj-2 has retired
      if (jj >= 2 && !mbar_wait_warp(&p_free[st], ((jj >> 1) - 1) & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) { ok = false; break; }
      const float mc = (m_used == -INFINITY) ? 0.f : m_used * c;
      const bool dead = m_used == -INFINITY;          // nothing visible yet: every probability of this tile is zero
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
      if (full) {
#pragma unroll
        for (int i0 = 0; i0 < KT; i0 += 2) {
          const float p0 = exp2f(__uint_as_float(sv[i0]) * c - mc);
          const float p1 = exp2f(__uint_as_float(sv[i0 + 1]) * c - mc);
          ps4[(i0 >> 1) & 3] += p0 + p1;
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          sv[i0 >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
      } else {
#pragma unroll
        for (int i0 = 0; i0 < KT; i0 += 2) {
          const float p0 = (!dead && i0 < limit && i0 >= lo) ? exp2f(__uint_as_float(sv[i0]) * c - mc) : 0.f;
          const float p1 = (!dead && i0 + 1 < limit && i0 + 1 >= lo) ? exp2f(__uint_as_float(sv[i0 + 1]) * c - mc) : 0.f;
          ps4[(i0 >> 1) & 3] += p0 + p1;
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          sv[i0 >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      l_run += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
#pragma unroll
      for (int cc = 0; cc < KT / 2; cc += 32) tmem_st32(tP0 + st * (KT / 2) + lane_sel + cc, sv + cc);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[st]);
    }
    // the last P V completes the output
    if (ok && !mbar_wait_warp(&p_free[(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue))
      ok = false;
    tc_fence_after();
    if (ok) {      // warp-uniform: the TMEM loads are warp-collective, only the stores are per row
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.out + b * p.o_bs + static_cast<long long>(row) * p.o_ts + hq * HD;
#pragma unroll 1
      for (int cc = 0; cc < HD; cc += 32) {
        uint32_t ov[32];
        __syncwarp();   // lanes that skipped the stores rejoin before the collective load
        tmem_ld32(tO + lane_sel + cc, ov);
        tmem_ld_wait();
        if (row < p.S) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 w;
            __nv_bfloat162* wh = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              wh[e] = __floats2bfloat162_rn(__uint_as_float(ov[ch * 8 + 2 * e]) * inv, __uint_as_float(ov[ch * 8 + 2 * e + 1]) * inv);
            reinterpret_cast<uint4*>(orow + cc)[ch] = w;
          }
        }
      }
      if (p.lse && row < p.S)
        p.lse[(static_cast<long long>(b) * p.Hq + hq) * p.S + row] = (l_run > 0.f) ? m_used * p.scale + logf(l_run) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

template <int HD, int KT>
const char* launch_tc3(const FlashArgs& a, void* vt_ws, int* status, cudaStream_t stream) {
  using C = Tc3Cfg<HD, KT>;
  const int s_pad = (a.Sk + 63) / 64 * 64;
  constexpr int tsm = 64 * (HD + 2) * 2;
  transpose_v_hd_kernel<HD><<<dim3(s_pad / 64, a.Hkv, a.B), 256, tsm, stream>>>(static_cast<const __nv_bfloat16*>(a.v), a.v_bs, a.v_ts,
                                                                               static_cast<__nv_bfloat16*>(vt_ws), a.Sk, s_pad, a.Hkv);
  count_launch();
  CUtensorMap tmQ, tmK, tmVt;
  if (!make_map_2d(&tmQ, a.q, static_cast<long long>(a.B) * a.Sq, static_cast<long long>(a.Hq) * HD, a.q_ts, FT))
    return "flash_fwd_tc: tensor map for Q failed";
  if (!make_map_2d(&tmK, a.k, static_cast<long long>(a.B) * a.Sk, static_cast<long long>(a.Hkv) * HD, a.k_ts, KT))
    return "flash_fwd_tc: tensor map for K failed";
  if (!make_map_2d(&tmVt, vt_ws, static_cast<long long>(a.B) * a.Hkv * HD, s_pad, s_pad, HD))
    return "flash_fwd_tc: tensor map for V^T failed";
  FlashTcParams p{};
  p.out = static_cast<__nv_bfloat16*>(a.o); p.o_bs = a.o_bs; p.o_ts = a.o_ts; p.lse = a.lse;
  p.B = a.B; p.S = a.Sq; p.Hq = a.Hq; p.Hkv = a.Hkv; p.scale = a.scale; p.status = status;
  auto kern = flash_fwd_tc3_kernel<HD, KT>;
  if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) == cudaSuccess))
    return "flash_fwd_tc: cannot reserve shared memory";
  dim3 grid((a.Sq + FT - 1) / FT, a.Hq, a.B);
  kern<<<grid, 192, C::SMEM, stream>>>(tmQ, tmK, tmVt, p, a.window);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "flash_fwd_tc launch failed";
}

}  // namespace

bool flash_fwd_tc_supported(const FlashArgs& a) {
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return (a.D == 128 || a.D == 256) && a.causal && a.window >= 0 && a.q_offset == 0 && a.Sq == a.Sk && a.Sq >= 1 && a.Hq % a.Hkv == 0 &&
         a.q_bs == static_cast<long long>(a.Sq) * a.q_ts && a.k_bs == static_cast<long long>(a.Sk) * a.k_ts &&
         (a.q_ts % 8) == 0 && (a.k_ts % 8) == 0 && (a.v_ts % 2) == 0 && (a.v_bs % 2) == 0 && (a.o_ts % 8) == 0 &&
         (a.o_bs % 8) == 0 && al16(a.q) && al16(a.k) && al16(a.o) && (reinterpret_cast<uintptr_t>(a.v) & 3) == 0;
}

size_t flash_fwd_tc_workspace_elems(const FlashArgs& a) {
  const long long s_pad = (a.Sk + 63) / 64 * 64;
  return static_cast<size_t>(a.B) * a.Hkv * a.D * s_pad;
}

// `vt_ws`: bf16 workspace of flash_fwd_tc_workspace_elems(a) elements, 16-byte aligned
const char* flash_fwd_tc(const FlashArgs& a, void* vt_ws, int* status, cudaStream_t stream, int form) {
  if (!flash_fwd_tc_supported(a)) return "flash_fwd_tc: unsupported arguments";
  if (a.B == 0) return nullptr;
  if (a.D == 256) return launch_tc3<256, 64>(a, vt_ws, status, stream);
  if (a.window > 0) return launch_tc3<128, 128>(a, vt_ws, status, stream);
  const int s_pad = (a.Sk + 63) / 64 * 64;
  transpose_v_kernel<<<dim3(s_pad / 64, a.Hkv, a.B), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(a.v), a.v_bs, a.v_ts,
                                                                     static_cast<__nv_bfloat16*>(vt_ws), a.Sk, s_pad, a.Hkv);
  count_launch();
  CUtensorMap tmQ, tmK, tmVt;
  if (!make_map_2d(&tmQ, a.q, static_cast<long long>(a.B) * a.Sq, static_cast<long long>(a.Hq) * FD, a.q_ts, FT))
    return "flash_fwd_tc: tensor map for Q failed";
  if (!make_map_2d(&tmK, a.k, static_cast<long long>(a.B) * a.Sk, static_cast<long long>(a.Hkv) * FD, a.k_ts, FT))
    return "flash_fwd_tc: tensor map for K failed";
  if (!make_map_2d(&tmVt, vt_ws, static_cast<long long>(a.B) * a.Hkv * FD, s_pad, s_pad, FT))
    return "flash_fwd_tc: tensor map for V^T failed";
  FlashTcParams p{};
  p.out = static_cast<__nv_bfloat16*>(a.o); p.o_bs = a.o_bs; p.o_ts = a.o_ts; p.lse = a.lse;
  p.B = a.B; p.S = a.Sq; p.Hq = a.Hq; p.Hkv = a.Hkv; p.scale = a.scale; p.status = status;
  constexpr int smem = 6 * TILE + 1024 + 256, smem2 = 7 * TILE + 1024 + 256, smem3 = 5 * TILE + 1024 + 256;
  if (!FERRL_ONCE_PER_DEVICE(
          cudaFuncSetAttribute(flash_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) == cudaSuccess &&
          cudaFuncSetAttribute(flash_fwd_tc2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) == cudaSuccess &&
          cudaFuncSetAttribute(flash_fwd_tc2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem3) == cudaSuccess))
    return "flash_fwd_tc: cannot reserve shared memory";
  dim3 grid((a.Sq + FT - 1) / FT, a.Hq, a.B);
  // form 0: output in registers; 1: output in TMEM, P through shared memory; 2: output and P in TMEM
  if (form == 2) flash_fwd_tc2_kernel<true><<<grid, 192, smem3, stream>>>(tmQ, tmK, tmVt, p);
  else if (form == 1) flash_fwd_tc2_kernel<false><<<grid, 192, smem2, stream>>>(tmQ, tmK, tmVt, p);
  else flash_fwd_tc_kernel<<<grid, 192, smem, stream>>>(tmQ, tmK, tmVt, p);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "flash_fwd_tc launch failed";
}

}  // namespace ferrl
