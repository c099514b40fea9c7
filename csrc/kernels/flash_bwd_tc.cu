// Causal flash-attention backward on the 5th-generation tensor cores (head_dim 128, optional sliding window).
//
// Two kernels, both deterministic (no floating-point atomics; every accumulator lives in TMEM and is
// summed in a fixed order):
//
//   flash_bwd_dq_kernel   one CTA per 128 query rows of one head, walks the key tiles j <= i:
//                           S = Q K_j^T, dP = dO V_j^T            (tcgen05, fp32 in TMEM)
//                           dS = P o (dP - delta) * scale          (softmax warps, P = exp(S*scale - lse))
//                           dQ += dS K_j                          (accumulated in TMEM across j)
//   flash_bwd_dkv_kernel  one CTA per 128 keys of one KV head, walks every query head of the group
//                         and the 64-row query tiles at or below the diagonal, in transposed form so
//                         that a thread owns a key:
//                           S^T = K Q_i^T, dP^T = V dO_i^T
//                           P^T, dS^T written to shared memory as K-major A operands
//                           dV += P^T dO_i,  dK += dS^T Q_i        (accumulated in TMEM across tiles and heads)
//
// With a window of w keys (query i sees keys (i - w, i]) the dQ kernel starts at the first key tile any of its
// rows sees and the dK/dV kernel stops at the last query tile that still has one of its keys in the window; only
// tiles cut by the diagonal or by the window's lower edge take the masked path.
//
// Every operand is a natural-layout tile written by TMA with the 128-byte swizzle (no cluster
// multicast).  Where the contraction runs over the tile's row index (dS K_j, P^T dO, dS^T Q) the
// B operand is read through an MN-major shared-memory descriptor, so no transposed copies of
// Q, K or dO are needed.  Warp roles: 0 TMA producer, 1 MMA issuer, 2-9 eight softmax warps (two
// threads per TMEM lane, each taking half of the tile's columns).  Every wait is bounded.
//
// Reference behaviour: the gradient of the eager GQA attention in crates/ferrl/src/dense.rs
// (candle autograd through softmax(QK^T)V); the warp-level kernel in flash_attn.cu stays as the
// path for other head dims, windows and offsets.
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

constexpr int FD = 128;                    // head dim
constexpr int FT = 128;                    // rows of a full tile
constexpr int QH = 64;                     // query rows per tile in the dK/dV kernel
constexpr int ATOM128 = FT * 64 * 2;       // [128 rows x 64 cols] swizzle atom: 16 KB
constexpr int TILE128 = 2 * ATOM128;       // [128 x 128] bf16: 32 KB
constexpr int ATOM64 = QH * 64 * 2;        // [64 rows x 64 cols]: 8 KB
constexpr int TILE64 = 2 * ATOM64;         // [64 x 128] bf16: 16 KB
constexpr int NST = 4;                     // Q/dO ring depth of the dK/dV kernel
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kBMajorMN = 1u << 16;   // instruction descriptor: B operand is MN-major
constexpr int BWD_THREADS = 320;

struct FlashBwdTcParams {
  const float2* stats;   // [B, Hq, S_pad] per query row: {lse * log2(e), rowsum(O o dO)}, zeros for the padding rows
  int S_pad;             // S rounded up to 128
  __nv_bfloat16* dq; long long dq_bs, dq_ts;
  __nv_bfloat16* dk; long long dk_bs, dk_ts;
  __nv_bfloat16* dv; long long dv_bs, dv_ts;
  int B, S, Hq, Hkv;
  float scale;
  int window;            // 0: plain causal; w > 0: query i sees keys (i - w, i]
  int* status;
  unsigned long long* debug;   // optional globaltimer stamps of CTA (0,0,0) of the dQ kernel: [step][8]
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// stats[b, h, s] = {lse[b, h, s] * log2(e), sum_d o[b, s, h, d] * do[b, s, h, d]} for s < S, zeros for the
// padding rows up to S_pad; one warp per row.  The padded, interleaved layout lets the dK/dV kernel
// fetch the 64 rows of a query tile with one 512-byte bulk copy per step.
__global__ void flash_stats_kernel(const __nv_bfloat16* __restrict__ o, long long o_bs, long long o_ts,
                                   const __nv_bfloat16* __restrict__ d_o, long long do_bs, long long do_ts,
                                   const float* __restrict__ lse, float2* __restrict__ stats, int B, int S, int S_pad, int Hq) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(B) * S_pad * Hq) return;
  const int h = static_cast<int>(w % Hq);
  const long long bs = w / Hq;
  const int s = static_cast<int>(bs % S_pad), b = static_cast<int>(bs / S_pad);
  float2* dst = stats + (static_cast<long long>(b) * Hq + h) * S_pad + s;
  if (s >= S) {
    if (lane == 0) *dst = make_float2(0.f, 0.f);
    return;
  }
  const uint2 ov = *reinterpret_cast<const uint2*>(o + b * o_bs + s * o_ts + h * FD + lane * 4);
  const uint2 dv = *reinterpret_cast<const uint2*>(d_o + b * do_bs + s * do_ts + h * FD + lane * 4);
  const float2 o0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov.x));
  const float2 o1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ov.y));
  const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.x));
  const float2 d1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.y));
  float acc = o0.x * d0.x + o0.y * d0.y + o1.x * d1.x + o1.y * d1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) *dst = make_float2(lse[(static_cast<long long>(b) * Hq + h) * S + s] * kLog2e, acc);
}

// ------------------------------------------------------------------------------------------ dQ
// K_j is needed from its S MMA until its dQ MMA, the last of the step, so the K ring is three deep
// (with two, the load of K_{j+2} could only start when S_{j+2} already wants it); V_j is needed by
// dP alone, early in the step, and has a single buffer that is refilled during the rest of the step.
constexpr int KRING = 3;
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    FlashBwdTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                      // 32 KB
  uint8_t* sdO = sQ + TILE128;             // 32 KB
  uint8_t* sK = sdO + TILE128;             // KRING x 32 KB
  uint8_t* sV = sK + KRING * TILE128;      // 32 KB
  uint8_t* sdS = sV + TILE128;             // 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + TILE128);
  uint64_t* qdo_full = bars;               // [1]
  uint64_t* k_full = bars + 1;             // [3]
  uint64_t* k_empty = bars + 4;            // [3]
  uint64_t* v_full = bars + 7;             // [1]
  uint64_t* v_empty = bars + 8;            // [1]
  uint64_t* s_full = bars + 9;             // S of tile j is in TMEM
  uint64_t* dp_full = bars + 10;           // dP of tile j is in TMEM
  uint64_t* sdp_empty = bars + 11;         // all softmax warps hold tile j's S and dP in registers
  uint64_t* ds_full = bars + 12;           // dS of tile j is in shared memory
  uint64_t* ds_free = bars + 13;           // the dQ MMAs reading dS have retired
  uint64_t* dq_full = bars + 14;           // every dQ MMA has retired
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.S + FT - 1) / FT;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);     // longest rows first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int hk = hq / (p.Hq / p.Hkv);
  const int q0 = qt * FT;
  const int j_lo = p.window > 0 ? max(0, q0 - p.window + 1) / FT : 0;   // first key tile any row of this CTA sees
  const int n_kv = qt + 1 - j_lo;                                        // steps j = 0 .. n_kv-1 walk key tiles j_lo + j
  unsigned long long* dbg = (p.debug && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.debug : nullptr;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < KRING; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(sdp_empty, 8);
    mbar_init(ds_full, 8);
    mbar_init(ds_free, 1);
    mbar_init(dq_full, 1);
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
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdQ = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(qdo_full, 2 * TILE128);
      tma_load_2d(sQ, &tmQ, qdo_full, hq * FD, b * p.S + q0);
      tma_load_2d(sQ + ATOM128, &tmQ, qdo_full, hq * FD + 64, b * p.S + q0);
      tma_load_2d(sdO, &tmdO, qdo_full, hq * FD, b * p.S + q0);
      tma_load_2d(sdO + ATOM128, &tmdO, qdo_full, hq * FD + 64, b * p.S + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j % KRING;
        const uint32_t ph = (j / KRING) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_expect_tx(&k_full[st], TILE128);
        tma_load_2d(sK + st * TILE128, &tmK, &k_full[st], hk * FD, b * p.S + (j_lo + j) * FT);
        tma_load_2d(sK + st * TILE128 + ATOM128, &tmK, &k_full[st], hk * FD + 64, b * p.S + (j_lo + j) * FT);
        if (!mbar_wait(v_empty, (j & 1) ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_expect_tx(v_full, TILE128);
        tma_load_2d(sV, &tmV, v_full, hk * FD, b * p.S + (j_lo + j) * FT);
        tma_load_2d(sV + ATOM128, &tmV, v_full, hk * FD + 64, b * p.S + (j_lo + j) * FT);
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(10000);   // let copies in flight land before shared memory goes away
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA warp: all lanes walk the loop, one issues
    constexpr uint32_t idesc = make_idesc_bf16(128, 128);
    const uint64_t dq_desc = make_smem_desc(smem_u32(sQ)), ddo_desc = make_smem_desc(smem_u32(sdO));
    const uint64_t ds_desc = make_smem_desc(smem_u32(sdS));
    const bool stamp = dbg && lane == 0;
    auto issue_sdp = [&](int j) -> bool {
      const int st = j % KRING;
      if (!mbar_wait_warp(&k_full[st], (j / KRING) & 1, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
      if (j > 0 && !mbar_wait_warp(sdp_empty, (j - 1) & 1, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
      tc_fence_after();
      if (stamp) dbg[j * 12 + 8] = globaltimer_ns();
      const uint64_t dk = make_smem_desc(smem_u32(sK + st * TILE128)), dv_ = make_smem_desc(smem_u32(sV));
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < FD / 16; ++k) {
          const uint32_t off = (k >> 2) * ATOM128 + (k & 3) * 32;
          umma(tS, desc_adv(dq_desc, off), desc_adv(dk, off), idesc, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
      }
      __syncwarp();
      // V has a single buffer that is refilled while S is computed: wait for it only now
      if (!mbar_wait_warp(v_full, j & 1, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < FD / 16; ++k) {
          const uint32_t off = (k >> 2) * ATOM128 + (k & 3) * 32;
          umma(tdP, desc_adv(ddo_desc, off), desc_adv(dv_, off), idesc, k > 0 ? 1u : 0u);
        }
        umma_commit(dp_full);
        umma_commit(v_empty);
      }
      __syncwarp();
      if (stamp) dbg[j * 12 + 5] = globaltimer_ns();
      return true;
    };
    bool ok = mbar_wait_warp(qdo_full, 0, abort_flag, p.status, kStatusWaitTimeoutMma);
    if (ok) ok = issue_sdp(0);
    for (int j = 0; j < n_kv && ok; ++j) {
      if (j + 1 < n_kv) ok = issue_sdp(j + 1);
      if (!ok) break;
      const int st = j % KRING;
      if (!mbar_wait_warp(ds_full, j & 1, abort_flag, p.status, kStatusWaitTimeoutMma)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (stamp) dbg[j * 12 + 6] = globaltimer_ns();
      const uint64_t dkm = make_smem_desc_mn(smem_u32(sK + st * TILE128), ATOM128);
      const uint32_t acc0 = j > 0 ? 1u : 0u;
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < FT / 16; ++k)     // contraction over the tile's 128 keys
          umma(tdQ, desc_adv(ds_desc, (k >> 2) * ATOM128 + (k & 3) * 32), desc_adv(dkm, k * 2048), idesc | kBMajorMN,
               k > 0 ? 1u : acc0);
        umma_commit(ds_free);
        umma_commit(&k_empty[st]);
      }
      __syncwarp();
      if (stamp) dbg[j * 12 + 7] = globaltimer_ns();
    }
    if (ok && elect_one()) umma_commit(dq_full);
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax warps: thread = (query row, half of the keys)
    const int qd = warp & 3, half = (warp - 2) >> 2;
    const int r = qd * 32 + lane;
    const int row = q0 + r;
    const uint32_t lane_sel = static_cast<uint32_t>(qd * 32) << 16;
    const float c = p.scale * kLog2e;
    const float2 st2 = p.stats[(static_cast<long long>(b) * p.Hq + hq) * p.S_pad + row];   // padded: no guard needed
    const float lse_c = st2.x, dlt = st2.y;
    const bool rows_ok = __all_sync(0xffffffffu, row < p.S);    // every row of this warp exists
    const bool stamp = dbg && warp == 2 && lane == 0;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait_warp(s_full, j & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue) ||
          !mbar_wait_warp(dp_full, j & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (stamp) dbg[j * 12 + 0] = globaltimer_ns();
      uint32_t sv[64], dv[64];
      tmem_ld32(tS + lane_sel + half * 64, sv);
      tmem_ld32(tS + lane_sel + half * 64 + 32, sv + 32);
      tmem_ld32(tdP + lane_sel + half * 64, dv);
      tmem_ld32(tdP + lane_sel + half * 64 + 32, dv + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sdp_empty);
      if (stamp) dbg[j * 12 + 1] = globaltimer_ns();
      // dS without the softmax scale (it is applied once to dQ at the end), packed to bf16 in place
      uint32_t w[32];
      const int ja = j_lo + j;                // key tile of this step
      // warp-uniform: a tile strictly below the diagonal and above the window's lower edge needs no mask
      if (ja < qt && rows_ok && (p.window == 0 || q0 + FT - p.window <= ja * FT + half * 64)) {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float d0 = exp2f(__uint_as_float(sv[2 * e]) * c - lse_c) * (__uint_as_float(dv[2 * e]) - dlt);
          const float d1 = exp2f(__uint_as_float(sv[2 * e + 1]) * c - lse_c) * (__uint_as_float(dv[2 * e + 1]) - dlt);
          w[e] = pack_bf16(d0, d1);
        }
      } else {
        const int k0 = ja * FT + half * 64;
        int nvalid = row < p.S ? (ja == qt ? row - k0 + 1 : 64) : 0;    // keys k0 .. k0+nvalid-1 are at or before the query
        nvalid = max(0, min(64, nvalid));
        const int lo = p.window > 0 ? row - p.window + 1 - k0 : -(1 << 30);   // keys below k0+lo have left the window
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float d0 = 0.f, d1 = 0.f;
          if (2 * e < nvalid && 2 * e >= lo) d0 = exp2f(__uint_as_float(sv[2 * e]) * c - lse_c) * (__uint_as_float(dv[2 * e]) - dlt);
          if (2 * e + 1 < nvalid && 2 * e + 1 >= lo) d1 = exp2f(__uint_as_float(sv[2 * e + 1]) * c - lse_c) * (__uint_as_float(dv[2 * e + 1]) - dlt);
          w[e] = pack_bf16(d0, d1);
        }
      }
      if (stamp) dbg[j * 12 + 2] = globaltimer_ns() + (w[0] == 0xdeadbeefu ? 1 : 0);
      if (j >= 1 && !mbar_wait_warp(ds_free, (j - 1) & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) {
        ok = false;
        break;
      }
      uint8_t* drow = sdS + half * ATOM128 + r * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        *reinterpret_cast<uint4*>(drow + ((ch ^ (r & 7)) << 4)) = make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
      if (stamp) dbg[j * 12 + 4] = globaltimer_ns();
    }
    if (ok && !mbar_wait_warp(dq_full, 0, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) ok = false;
    tc_fence_after();
    if (ok) {      // warp-uniform: the TMEM loads are warp-collective, only the stores are per row
      __nv_bfloat16* orow = p.dq + b * p.dq_bs + static_cast<long long>(row) * p.dq_ts + hq * FD + half * 64;
      const float sc = p.scale;
#pragma unroll 1
      for (int cc = 0; cc < 64; cc += 32) {
        uint32_t ov[32];
        __syncwarp();   // lanes that skipped the stores rejoin before the collective load
        tmem_ld32(tdQ + lane_sel + half * 64 + cc, ov);
        tmem_ld_wait();
        if (row >= p.S) continue;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint4 w4;
          w4.x = pack_bf16(__uint_as_float(ov[ch * 8 + 0]) * sc, __uint_as_float(ov[ch * 8 + 1]) * sc);
          w4.y = pack_bf16(__uint_as_float(ov[ch * 8 + 2]) * sc, __uint_as_float(ov[ch * 8 + 3]) * sc);
          w4.z = pack_bf16(__uint_as_float(ov[ch * 8 + 4]) * sc, __uint_as_float(ov[ch * 8 + 5]) * sc);
          w4.w = pack_bf16(__uint_as_float(ov[ch * 8 + 6]) * sc, __uint_as_float(ov[ch * 8 + 7]) * sc);
          reinterpret_cast<uint4*>(orow + cc)[ch] = w4;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ------------------------------------------------------------------------------------------ dK, dV
__global__ void __launch_bounds__(BWD_THREADS, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmQ64, const __grid_constant__ CUtensorMap tmdO64,
                     FlashBwdTcParams p) {
  // The four-deep Q/dO ring leaves no room for alignment slack: the dynamic shared memory is declared
  // 1024-byte aligned (the swizzled tiles need it) and the kernel refuses to run if it is not.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, kStatusOk, kStatusBadShape);
    return;
  }
  uint8_t* sK = smem;                       // 32 KB, resident
  uint8_t* sV = sK + TILE128;               // 32 KB, resident
  uint8_t* sQ = sV + TILE128;               // NST x 16 KB
  uint8_t* sdO = sQ + NST * TILE64;         // NST x 16 KB
  uint8_t* sPt = sdO + NST * TILE64;        // [128 keys x 64 queries] 16 KB
  uint8_t* sdSt = sPt + ATOM128;            // 16 KB
  float2* sStat = reinterpret_cast<float2*>(sdSt + ATOM128);   // NST x 64 rows of {lse*log2e, delta}
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdSt + ATOM128 + NST * QH * 8);
  uint64_t* kv_full = bars;                 // [1]
  uint64_t* qdo_full = bars + 1;            // [NST]
  uint64_t* qdo_empty = bars + 1 + NST;     // [NST]
  uint64_t* s_full = bars + 1 + 2 * NST;
  uint64_t* dp_full = s_full + 1;
  uint64_t* sdp_empty = s_full + 2;
  uint64_t* pds_full = s_full + 3;
  uint64_t* pds_free = s_full + 4;
  uint64_t* out_full = s_full + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x;                                   // key tile; tile 0 has the most work and runs first
  const int hk = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int n64 = (p.S + QH - 1) / QH;
  const int i_lo = 2 * kt;                                     // first 64-row query tile that can see these keys
  // last 64-row query tile that still has one of these keys inside its window
  const int i_hi = p.window > 0 ? min(n64 - 1, (kt * FT + FT - 1 + p.window - 1) / QH) : n64 - 1;
  const int cnt = i_hi - i_lo + 1;                             // query tiles per head (>= 1)
  const int T = G * cnt;
  unsigned long long* dbg = (p.debug && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.debug + 512 : nullptr;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < NST; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(sdp_empty, 8);
    mbar_init(pds_full, 8);
    mbar_init(pds_free, 1);
    mbar_init(out_full, 1);
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
  const uint32_t tSt = tmem_base, tdPt = tmem_base + 64, tdV = tmem_base + 128, tdK = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * TILE128);
      tma_load_2d(sK, &tmK, kv_full, hk * FD, b * p.S + kt * FT);
      tma_load_2d(sK + ATOM128, &tmK, kv_full, hk * FD + 64, b * p.S + kt * FT);
      tma_load_2d(sV, &tmV, kv_full, hk * FD, b * p.S + kt * FT);
      tma_load_2d(sV + ATOM128, &tmV, kv_full, hk * FD + 64, b * p.S + kt * FT);
      for (int t = 0; t < T; ++t) {
        const int st = t % NST;
        const uint32_t ph = (t / NST) & 1;
        const int hq = hk * G + t / cnt;
        const int q0 = (i_lo + t % cnt) * QH;
        if (!mbar_wait(&qdo_empty[st], ph ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) break;
        mbar_expect_tx(&qdo_full[st], 2 * TILE64 + QH * 8);
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(sStat + st * QH)),
                       "l"(reinterpret_cast<uint64_t>(p.stats + (static_cast<long long>(b) * p.Hq + hq) * p.S_pad + q0)),
                       "r"(QH * 8), "r"(smem_u32(&qdo_full[st]))
                     : "memory");
        tma_load_2d(sQ + st * TILE64, &tmQ64, &qdo_full[st], hq * FD, b * p.S + q0);
        tma_load_2d(sQ + st * TILE64 + ATOM64, &tmQ64, &qdo_full[st], hq * FD + 64, b * p.S + q0);
        tma_load_2d(sdO + st * TILE64, &tmdO64, &qdo_full[st], hq * FD, b * p.S + q0);
        tma_load_2d(sdO + st * TILE64 + ATOM64, &tmdO64, &qdo_full[st], hq * FD + 64, b * p.S + q0);
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(10000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA warp: all lanes walk the loop, one issues
    constexpr uint32_t idesc_s = make_idesc_bf16(128, QH);
    constexpr uint32_t idesc_acc = make_idesc_bf16(128, 128) | kBMajorMN;
    const uint64_t dk_desc = make_smem_desc(smem_u32(sK)), dv_desc = make_smem_desc(smem_u32(sV));
    const uint64_t dpt_desc = make_smem_desc(smem_u32(sPt)), dst_desc = make_smem_desc(smem_u32(sdSt));
    auto issue_sdp = [&](int t) -> bool {
      const int st = t % NST;
      const uint32_t ph = (t / NST) & 1;
      if (!mbar_wait_warp(&qdo_full[st], ph, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
      if (t > 0 && !mbar_wait_warp(sdp_empty, (t - 1) & 1, abort_flag, p.status, kStatusWaitTimeoutMma)) return false;
      tc_fence_after();
      if (dbg && lane == 0 && t < 40) dbg[t * 12 + 8] = globaltimer_ns();
      const uint64_t dq_ = make_smem_desc(smem_u32(sQ + st * TILE64)), ddo = make_smem_desc(smem_u32(sdO + st * TILE64));
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < FD / 16; ++ks)
          umma(tSt, desc_adv(dk_desc, (ks >> 2) * ATOM128 + (ks & 3) * 32), desc_adv(dq_, (ks >> 2) * ATOM64 + (ks & 3) * 32), idesc_s,
               ks > 0 ? 1u : 0u);
        umma_commit(s_full);
#pragma unroll
        for (int ks = 0; ks < FD / 16; ++ks)
          umma(tdPt, desc_adv(dv_desc, (ks >> 2) * ATOM128 + (ks & 3) * 32), desc_adv(ddo, (ks >> 2) * ATOM64 + (ks & 3) * 32), idesc_s,
               ks > 0 ? 1u : 0u);
        umma_commit(dp_full);
      }
      __syncwarp();
      if (dbg && lane == 0 && t < 40) dbg[t * 12 + 5] = globaltimer_ns();
      return true;
    };
    bool ok = mbar_wait_warp(kv_full, 0, abort_flag, p.status, kStatusWaitTimeoutMma);
    if (ok) ok = issue_sdp(0);
    for (int t = 0; t < T && ok; ++t) {
      if (t + 1 < T) ok = issue_sdp(t + 1);
      if (!ok) break;
      const int st = t % NST;
      if (!mbar_wait_warp(pds_full, t & 1, abort_flag, p.status, kStatusWaitTimeoutMma)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (dbg && lane == 0 && t < 40) dbg[t * 12 + 6] = globaltimer_ns();
      const uint64_t ddom = make_smem_desc_mn(smem_u32(sdO + st * TILE64), ATOM64);
      const uint64_t dqm = make_smem_desc_mn(smem_u32(sQ + st * TILE64), ATOM64);
      const uint32_t acc0 = t > 0 ? 1u : 0u;
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < QH / 16; ++ks)       // contraction over the tile's 64 queries
          umma(tdV, desc_adv(dpt_desc, ks * 32), desc_adv(ddom, ks * 2048), idesc_acc, ks > 0 ? 1u : acc0);
#pragma unroll
        for (int ks = 0; ks < QH / 16; ++ks)
          umma(tdK, desc_adv(dst_desc, ks * 32), desc_adv(dqm, ks * 2048), idesc_acc, ks > 0 ? 1u : acc0);
        umma_commit(pds_free);
        umma_commit(&qdo_empty[st]);
      }
      __syncwarp();
      if (dbg && lane == 0 && t < 40) dbg[t * 12 + 7] = globaltimer_ns();
    }
    if (ok && elect_one()) umma_commit(out_full);
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax warps: thread = (key, half of the tile's queries)
    const int qd = warp & 3, half = (warp - 2) >> 2;
    const int r = qd * 32 + lane;
    const int key = kt * FT + r;
    const uint32_t lane_sel = static_cast<uint32_t>(qd * 32) << 16;
    const float c = p.scale * kLog2e;
    bool ok = true;
    for (int t = 0; t < T; ++t) {
      const int hq = hk * G + t / cnt;
      const int qbase = (i_lo + t % cnt) * QH + half * 32;
      if (!mbar_wait_warp(s_full, t & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue) ||
          !mbar_wait_warp(dp_full, t & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const float2* st_row = sStat + (t % NST) * QH + half * 32;     // landed with this step's Q/dO tile (same barrier as S's operands)
      const bool stamp = dbg && warp == 2 && lane == 0 && t < 40;
      if (stamp) dbg[t * 12 + 0] = globaltimer_ns();
      uint32_t sv[32], dv[32];
      tmem_ld32(tSt + lane_sel + half * 32, sv);
      tmem_ld32(tdPt + lane_sel + half * 32, dv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sdp_empty);
      if (stamp) dbg[t * 12 + 1] = globaltimer_ns();
      // P^T and dS^T (without the softmax scale: it is applied once to dK at the end) as packed bf16
      uint32_t pw[16], dw[16];
      // warp-uniform: every query is real, at or after every key, and no key has left any query's window
      if (qbase >= kt * FT + FT - 1 && qbase + 32 <= p.S && (p.window == 0 || qbase + 31 - kt * FT < p.window)) {
#pragma unroll
        for (int e2 = 0; e2 < 16; ++e2) {
          const float4 s4 = *reinterpret_cast<const float4*>(st_row + 2 * e2);     // {lse, delta} of two queries (broadcast read)
          const float p0 = exp2f(__uint_as_float(sv[2 * e2]) * c - s4.x);
          const float p1 = exp2f(__uint_as_float(sv[2 * e2 + 1]) * c - s4.z);
          pw[e2] = pack_bf16(p0, p1);
          dw[e2] = pack_bf16(p0 * (__uint_as_float(dv[2 * e2]) - s4.y), p1 * (__uint_as_float(dv[2 * e2 + 1]) - s4.w));
        }
      } else {
#pragma unroll
        for (int e2 = 0; e2 < 16; ++e2) {
          const float4 s4 = *reinterpret_cast<const float4*>(st_row + 2 * e2);
          const int q = qbase + 2 * e2;
          float p0 = 0.f, p1 = 0.f, d0 = 0.f, d1 = 0.f;
          if (q < p.S && key <= q && (p.window == 0 || q - key < p.window)) {
            p0 = exp2f(__uint_as_float(sv[2 * e2]) * c - s4.x);
            d0 = p0 * (__uint_as_float(dv[2 * e2]) - s4.y);
          }
          if (q + 1 < p.S && key <= q + 1 && (p.window == 0 || q + 1 - key < p.window)) {
            p1 = exp2f(__uint_as_float(sv[2 * e2 + 1]) * c - s4.z);
            d1 = p1 * (__uint_as_float(dv[2 * e2 + 1]) - s4.w);
          }
          pw[e2] = pack_bf16(p0, p1);
          dw[e2] = pack_bf16(d0, d1);
        }
      }
      if (stamp) dbg[t * 12 + 2] = globaltimer_ns() + (pw[0] == 0xdeadbeefu ? 1 : 0);
      if (t >= 1 && !mbar_wait_warp(pds_free, (t - 1) & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) {
        ok = false;
        break;
      }
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        const int gch = half * 4 + ch;
        const uint32_t off = r * 128 + ((gch ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(sPt + off) = make_uint4(pw[4 * ch], pw[4 * ch + 1], pw[4 * ch + 2], pw[4 * ch + 3]);
        *reinterpret_cast<uint4*>(sdSt + off) = make_uint4(dw[4 * ch], dw[4 * ch + 1], dw[4 * ch + 2], dw[4 * ch + 3]);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (stamp) dbg[t * 12 + 4] = globaltimer_ns();
    }
    if (ok && !mbar_wait_warp(out_full, 0, abort_flag, p.status, kStatusWaitTimeoutEpilogue)) ok = false;
    tc_fence_after();
    if (ok) {      // warp-uniform, as above
      __nv_bfloat16* vrow = p.dv + b * p.dv_bs + static_cast<long long>(key) * p.dv_ts + hk * FD + half * 64;
      __nv_bfloat16* krow = p.dk + b * p.dk_bs + static_cast<long long>(key) * p.dk_ts + hk * FD + half * 64;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = (which == 0 ? tdV : tdK) + lane_sel + half * 64;
        __nv_bfloat16* dst = which == 0 ? vrow : krow;
        const float sc = which == 0 ? 1.f : p.scale;
#pragma unroll 1
        for (int cc = 0; cc < 64; cc += 32) {
          uint32_t ov[32];
          __syncwarp();   // lanes that skipped the stores rejoin before the collective load
          tmem_ld32(src + cc, ov);
          tmem_ld_wait();
          if (key >= p.S) continue;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(ov[ch * 8 + 0]) * sc, __uint_as_float(ov[ch * 8 + 1]) * sc);
            w.y = pack_bf16(__uint_as_float(ov[ch * 8 + 2]) * sc, __uint_as_float(ov[ch * 8 + 3]) * sc);
            w.z = pack_bf16(__uint_as_float(ov[ch * 8 + 4]) * sc, __uint_as_float(ov[ch * 8 + 5]) * sc);
            w.w = pack_bf16(__uint_as_float(ov[ch * 8 + 6]) * sc, __uint_as_float(ov[ch * 8 + 7]) * sc);
            reinterpret_cast<uint4*>(dst + cc)[ch] = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

}  // namespace

size_t flash_bwd_tc_scratch_floats(const FlashArgs& a) {
  return static_cast<size_t>(a.B) * a.Hq * ((a.Sq + FT - 1) / FT * FT) * 2;
}

bool flash_bwd_tc_supported(const FlashArgs& a) {
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return a.D == FD && a.causal && a.window >= 0 && a.q_offset == 0 && a.Sq == a.Sk && a.Sq >= 1 && a.Hq % a.Hkv == 0 &&
         a.q_bs == static_cast<long long>(a.Sq) * a.q_ts && a.k_bs == static_cast<long long>(a.Sk) * a.k_ts &&
         a.v_bs == static_cast<long long>(a.Sk) * a.v_ts && a.do_bs == static_cast<long long>(a.Sq) * a.do_ts &&
         (a.q_ts % 8) == 0 && (a.k_ts % 8) == 0 && (a.v_ts % 8) == 0 && (a.do_ts % 8) == 0 && (a.o_ts % 4) == 0 &&
         (a.o_bs % 4) == 0 && (a.dq_ts % 8) == 0 && (a.dk_ts % 8) == 0 && (a.dv_ts % 8) == 0 && (a.dq_bs % 8) == 0 &&
         (a.dk_bs % 8) == 0 && (a.dv_bs % 8) == 0 && al16(a.q) && al16(a.k) && al16(a.v) && al16(a.d_o) && al16(a.dq) &&
         al16(a.dk) && al16(a.dv) && (reinterpret_cast<uintptr_t>(a.o) & 7) == 0;
}

// Needs a.lse from the forward and a.delta: fp32 scratch of flash_bwd_tc_scratch_floats(a) elements, 16-byte aligned.
const char* flash_bwd_tc(const FlashArgs& a, int* status, cudaStream_t stream) {
  if (!flash_bwd_tc_supported(a)) return "flash_bwd_tc: unsupported arguments";
  if (a.B == 0) return nullptr;
  const int s_pad = (a.Sq + FT - 1) / FT * FT;
  const long long rows = static_cast<long long>(a.B) * s_pad * a.Hq;
  float2* stats = reinterpret_cast<float2*>(a.delta);
  flash_stats_kernel<<<static_cast<unsigned>((rows * 32 + 255) / 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a.o), a.o_bs, a.o_ts, static_cast<const __nv_bfloat16*>(a.d_o), a.do_bs, a.do_ts,
      a.lse, stats, a.B, a.Sq, s_pad, a.Hq);
  count_launch();
  CUtensorMap tmQ, tmK, tmV, tmdO, tmQ64, tmdO64;
  const long long tok = static_cast<long long>(a.B) * a.Sq;
  if (!make_map_2d(&tmQ, a.q, tok, static_cast<long long>(a.Hq) * FD, a.q_ts, FT) ||
      !make_map_2d(&tmQ64, a.q, tok, static_cast<long long>(a.Hq) * FD, a.q_ts, QH) ||
      !make_map_2d(&tmK, a.k, tok, static_cast<long long>(a.Hkv) * FD, a.k_ts, FT) ||
      !make_map_2d(&tmV, a.v, tok, static_cast<long long>(a.Hkv) * FD, a.v_ts, FT) ||
      !make_map_2d(&tmdO, a.d_o, tok, static_cast<long long>(a.Hq) * FD, a.do_ts, FT) ||
      !make_map_2d(&tmdO64, a.d_o, tok, static_cast<long long>(a.Hq) * FD, a.do_ts, QH))
    return "flash_bwd_tc: tensor map failed";
  FlashBwdTcParams p{};
  p.stats = stats; p.S_pad = s_pad;
  p.dq = static_cast<__nv_bfloat16*>(a.dq); p.dq_bs = a.dq_bs; p.dq_ts = a.dq_ts;
  p.dk = static_cast<__nv_bfloat16*>(a.dk); p.dk_bs = a.dk_bs; p.dk_ts = a.dk_ts;
  p.dv = static_cast<__nv_bfloat16*>(a.dv); p.dv_bs = a.dv_bs; p.dv_ts = a.dv_ts;
  p.B = a.B; p.S = a.Sq; p.Hq = a.Hq; p.Hkv = a.Hkv; p.scale = a.scale; p.window = a.window; p.status = status; p.debug = a.debug;
  constexpr int smem_dq = 7 * TILE128 + 1024 + 256;
  constexpr int smem_dkv = 2 * TILE128 + 2 * NST * TILE64 + 2 * ATOM128 + NST * QH * 8 + 256;
  if (!FERRL_ONCE_PER_DEVICE(
          cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq) == cudaSuccess &&
          cudaFuncSetAttribute(flash_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dkv) == cudaSuccess))
    return "flash_bwd_tc: cannot reserve shared memory";
  const int n_t = (a.Sq + FT - 1) / FT;
  flash_bwd_dq_kernel<<<dim3(n_t, a.Hq, a.B), BWD_THREADS, smem_dq, stream>>>(tmQ, tmK, tmV, tmdO, p);
  count_launch();
  flash_bwd_dkv_kernel<<<dim3(n_t, a.Hkv, a.B), BWD_THREADS, smem_dkv, stream>>>(tmK, tmV, tmQ64, tmdO64, p);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "flash_bwd_tc launch failed";
}

}  // namespace ferrl
