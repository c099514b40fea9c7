// Decode-shaped bf16 projection for sm_100a:  out[M,N] = A[M,K] * B[N,K]^T  (+ residual | GLU),  M <= 128.
//
// A decode step multiplies one 128-row activation tile by every weight matrix of the model.  The
// weights stream from HBM exactly once, so the kernel is bound by how many bytes each SM pulls
// into shared memory; in a conventional tiling every CTA re-reads the activation tile for every
// weight tile it touches and that re-read traffic is between a third and a half of the fill.
// Here the activations are loaded ONCE per CTA and stay resident in TENSOR MEMORY:
//
//   * a cluster of S = 8 CTAs splits K: CTA r keeps its k-slice of the activation tile
//     ([128, <= 512] bf16 = 256 TMEM columns, row i in lane i, two bf16 per 32-bit column) for the
//     whole kernel; the epilogue threads read their rows from global memory once and write them
//     with tcgen05.st, and every tcgen05.mma takes its A operand from TMEM.  Shared memory is
//     left to the weight ring: 18 stages of 8 KB, enough bytes in flight per SM to cover the HBM
//     latency at full bandwidth;
//   * the cluster walks output tiles of BN = 64 weight rows; per tile a CTA streams only its
//     [64, k-slice] block of the weights through the TMA ring (no cluster multicast) and
//     accumulates into one of two TMEM accumulators;
//   * the S partial tiles are reduce-scattered through distributed shared memory: every CTA
//     owns 8 of the 64 columns, the peers store their fp32 partials of those columns into one of
//     two receive buffers (plain 16-byte stores, then one release-arrive per warp on the owner's
//     mbarrier), the owner adds the 8 partials in rank order (bit-reproducible) and writes its
//     columns.  Warp q of every CTA handles rows 32q..32q+31 on both sides, so the exchange is
//     synchronised per warp, and the exchange of tile i overlaps the main loop of tile i+1;
//   * K > 4096 does not fit one resident slice per CTA: the k range is cut into G groups, each
//     handled by its own clusters, whose fp32 partial outputs are summed (in group order) by a
//     small second kernel that also adds the residual.
//
// Warp roles: warp 0 TMA producer, warp 1 MMA issue (whole warp in the loop, elected lane
// issues), warps 2-5 activation load + epilogue.  Every mbarrier wait is bounded (2 s): on expiry
// the role records a status code, raises the CTA's abort flag and every role falls through to the
// common exit, where the cluster synchronises once and TMEM is released.  Launched as a
// programmatic dependent: the weight stream starts at once, only the activation load waits for
// the stream predecessor.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"
#include "tc_common.cuh"

namespace ferrl {

namespace {

using namespace tc;

constexpr int DG_BM = 128;
constexpr int DG_BN = 64;
constexpr int DG_BK = 64;
constexpr int DG_S = 8;                 // cluster size = k-split
constexpr int DG_RES = 8;               // resident activation k-blocks per CTA (8 x 32 TMEM columns)
constexpr int DG_STAGES = 14;           // weight ring, 8 KB per stage
constexpr int DG_NBUF = 2;              // exchange buffers in flight (tiles t .. t - DG_NBUF + 1)
constexpr int DG_THREADS = 192;
constexpr int DG_A_BYTES = DG_BM * DG_BK * 2;      // one activation k-block as TMA lands it: 16 KB
constexpr int DG_B_BYTES = DG_BN * DG_BK * 2;      // 8 KB
constexpr int DG_CHUNK = 2 * 32 * 16;              // one warp's partial for one peer: [2 runs][32 rows] float4 = 1 KB
constexpr int DG_RED_BYTES = (DG_S - 1) * 4 * DG_CHUNK;     // one receive (or staging) buffer: [slot][warp] chunks = 28 KB
constexpr int DG_SMEM = DG_STAGES * DG_B_BYTES + 2 * DG_NBUF * DG_RED_BYTES + 512 + 1024;
// the activations land (once, by TMA) in the tail of the dynamic shared memory: the receive and staging buffers and,
// where those are smaller than the resident slice, the last stages of the weight ring; none of that memory is in
// use before the first MMA (the producer holds back the overlapped stages until the rows are in tensor memory)
constexpr int DG_LAND_OFF = DG_STAGES * DG_B_BYTES + 2 * DG_NBUF * DG_RED_BYTES - DG_RES * (DG_BM * DG_BK * 2);
static_assert(DG_LAND_OFF >= 0 && DG_LAND_OFF % 1024 == 0, "landing zone must start on a swizzle-atom boundary");
constexpr int DG_LAND_STAGE = DG_LAND_OFF / DG_B_BYTES;   // first ring stage that the landing zone overlaps (>= DG_STAGES: none)
constexpr int DG_TMEM_COLS = 512;       // 256 columns of activations + two 64-column accumulators
constexpr int DG_ACC_COL = DG_RES * 32; // first accumulator column

struct DgParams {
  int M, N, K;
  int G, C;                 // k groups, clusters per group
  int kb_total, kb_group;   // k-blocks overall / per group
  int n_tiles;
  __nv_bfloat16* out; long long ldo;
  const __nv_bfloat16* residual; long long ldr;
  float* partial;           // [G, M, N] fp32 when G > 1
  int glu_act;
  int pdl;
  int* status;
  const __nv_bfloat16* A; long long lda;
  unsigned long long* debug;   // optional: globaltimer stamps of cluster 0 / rank 0 / warp 2 (see the epilogue)
};

__device__ __forceinline__ uint32_t dg_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t dg_mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void dg_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void dg_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void dg_cluster_sync() {
  dg_cluster_arrive();
  dg_cluster_wait();
}
// "I have consumed what you sent": the values read from the receive buffer have already been used when
// this executes, and nothing this thread wrote needs to be published with it, so the arrive carries no
// release (a release at cluster scope would first drain the thread's earlier global stores).
__device__ __forceinline__ void dg_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void dg_st_cluster_f4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Bulk copy from this CTA's shared memory into a peer's; the bytes are counted on an mbarrier of the peer, whose
// wait makes them visible there.  Runs on the copy engine: the issuing thread does not wait for it.
__device__ __forceinline__ void dg_bulk_to_peer(uint32_t dst_cluster_addr, uint32_t src_cta_addr, uint32_t bytes,
                                                uint32_t bar_cluster_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster_addr), "r"(src_cta_addr), "r"(bytes), "r"(bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void dg_tmem_st32(uint32_t taddr, const uint32_t* r) {
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
__device__ __forceinline__ void dg_tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// tcgen05.mma with the A operand in tensor memory (row i in lane i, two bf16 per 32-bit column)
__device__ __forceinline__ void dg_umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ bool dg_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait on a barrier that peers of the cluster signal; one answer for the whole warp.
__device__ __forceinline__ bool dg_wait_cluster_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                     int code) {
  bool ok = true;
  if (!dg_try_wait_cluster(bar, parity)) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (!dg_try_wait_cluster(bar, parity)) {
      if ((++spins & 0xff) == 0) {
        if (*abort_flag) { ok = false; break; }
        if (globaltimer_ns() - t0 > kWaitLimitNs) {
          *abort_flag = 1;
          atomicCAS(status, kStatusOk, code);
          ok = false;
          break;
        }
      }
    }
  }
  return __all_sync(0xffffffffu, ok);
}
// Column runs (two float4 = 8 accumulator columns) of the 64-column tile that cluster rank d owns.
// Plain: columns 8d .. 8d+7.  GLU: the weight rows come in groups of 16 (8 gate rows, then the 8 up
// rows of the same features); rank d owns 4 features: gate columns 16(d/2) + 4(d%2) .. +3 and the up
// columns 8 further on.
template <bool GLU> __device__ __forceinline__ constexpr int dg_run0(int d) { return GLU ? 16 * (d / 2) + 4 * (d % 2) : 8 * d; }
template <bool GLU> __device__ __forceinline__ constexpr int dg_run1(int d) { return GLU ? dg_run0<true>(d) + 8 : 8 * d + 4; }

template <bool GLU, bool HAS_RES, bool PARTIAL>
__global__ void __launch_bounds__(DG_THREADS, 1)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, DgParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* b_ring = smem;
  uint8_t* red = b_ring + DG_STAGES * DG_B_BYTES;        // [DG_NBUF][7 slots][4 warps] chunks, filled by the peers
  uint8_t* stg = red + DG_NBUF * DG_RED_BYTES;           // [DG_NBUF][7 peers][4 warps] chunks, my outgoing partials
  uint8_t* land = smem + DG_LAND_OFF;                    // activation landing zone (see DG_LAND_OFF)
  uint64_t* bars = reinterpret_cast<uint64_t*>(stg + DG_NBUF * DG_RED_BYTES);
  uint64_t* full = bars;                         // [DG_STAGES]
  uint64_t* empty = full + DG_STAGES;            // [DG_STAGES]
  uint64_t* acc_full = empty + DG_STAGES;        // [2]
  uint64_t* acc_empty = acc_full + 2;            // [2]
  uint64_t* a_land = acc_empty + 2;              // [1] the activation k-blocks have landed in shared memory
  uint64_t* a_ready = a_land + 1;                // [1] ... and have been moved to tensor memory
  uint64_t* red_full = a_ready + 1;              // [DG_NBUF][4 warps] the peers' partials of my columns have landed
  uint64_t* peers_free = red_full + 4 * DG_NBUF; // [DG_NBUF][4 warps] every peer has consumed what I sent into that buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(peers_free + 4 * DG_NBUF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(dg_cluster_rank());
  const int cluster_id = blockIdx.x / DG_S;
  const int g = cluster_id / p.C;                // k group
  const int c = cluster_id % p.C;                // cluster within the group
  const int kb_g0 = g * p.kb_group;
  const int kb_g1 = min(p.kb_total, kb_g0 + p.kb_group);
  const int kb_per = (kb_g1 - kb_g0 + DG_S - 1) / DG_S;
  const int kb_begin = min(kb_g1, kb_g0 + rank * kb_per);
  const int kb_cnt = min(kb_g1, kb_begin + kb_per) - kb_begin;       // 0 .. DG_RES
  const int my_tiles = c < p.n_tiles ? (p.n_tiles - c + p.C - 1) / p.C : 0;
  const bool work = kb_cnt > 0 && my_tiles > 0;  // a rank without k-blocks only contributes zeros to the exchange

  if (threadIdx.x == 0) pdl_trigger();
  if (threadIdx.x == 0) {
    for (int i = 0; i < DG_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);               // one arrive per epilogue warp
    }
    mbar_init(a_land, 1);
    mbar_init(a_ready, 4);
    for (int i = 0; i < 4 * DG_NBUF; ++i) {
      mbar_init(&red_full[i], 1);                // armed by the receiving warp; the data arrives as transaction bytes
      mbar_init(&peers_free[i], DG_S - 1);       // warp q of every peer
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(DG_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Peers signal into this CTA's barriers: every CTA of the cluster must have initialised them before
  // the first exchange.  Arrive now; each role waits where it first needs it.
  dg_cluster_arrive();

  if (warp == 0) {
    // ------------------------------------------------------------------ producer: the weight stream
    // The weights are never written by an earlier kernel of the stream, so nothing here waits for the
    // stream predecessor.
    dg_cluster_wait();
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      bool land_free = !work || DG_LAND_STAGE >= DG_STAGES;
      for (int t = 0; t < my_tiles && ok; ++t) {
        const int ni = c + t * p.C;
        for (int j = 0; j < kb_cnt; ++j) {
          if (!land_free && stage >= DG_LAND_STAGE) {
            if (!mbar_wait(a_ready, 0, abort_flag, p.status, kStatusWaitTimeoutProducer)) {
              ok = false;
              break;
            }
            land_free = true;
          }
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], DG_B_BYTES);
          tma_load_2d(b_ring + stage * DG_B_BYTES, &tmB, &full[stage], (kb_begin + j) * DG_BK, ni * DG_BN);
          if (++stage == DG_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    dg_cluster_wait();
    constexpr uint32_t idesc = make_idesc_bf16(DG_BM, DG_BN);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = work;
    if (ok) ok = mbar_wait_warp(a_ready, 0, abort_flag, p.status, kStatusWaitTimeoutMma);
    for (int t = 0; t < my_tiles && ok; ++t) {
      const int ab = t & 1;
      if (t >= 2) ok = mbar_wait_warp(&acc_empty[ab], ((t >> 1) - 1) & 1, abort_flag, p.status, kStatusWaitTimeoutMma);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + DG_ACC_COL + ab * DG_BN;
      for (int j = 0; j < kb_cnt; ++j) {
        ok = mbar_wait_warp(&full[stage], phase, abort_flag, p.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint64_t db = make_smem_desc(smem_u32(b_ring + stage * DG_B_BYTES));
        const uint32_t a_tmem = tmem_base + j * 32;
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < DG_BK / 16; ++k) dg_umma_ts(d_tmem, a_tmem + k * 8, desc_adv(db, k * 32), idesc, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[stage]);
        }
        __syncwarp();
        if (++stage == DG_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) {
        if (elect_one()) umma_commit(&acc_full[ab]);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ activation load, epilogue, exchange
    dg_cluster_wait();
    const int q = warp & 3;                         // TMEM lane quarter of this warp
    const int row = q * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const bool stamp = p.debug != nullptr && blockIdx.x == 0 && warp == 2 && lane == 0;
    if (stamp) p.debug[0] = globaltimer_ns();
    bool ok = true;
    if (work) {
      // The activations come from the stream predecessor.  One thread fetches my k-slice with TMA (128-byte
      // rows, 128B swizzle) into the landing zone; every thread then moves its own row into tensor memory:
      // 32 packed columns per k-block, zeros beyond M and K (TMA fills them).
      if (warp == 2 && lane == 0) {
        if (p.pdl) pdl_wait();
        mbar_expect_tx(a_land, kb_cnt * DG_A_BYTES);
        for (int j = 0; j < kb_cnt; ++j) tma_load_2d(land + j * DG_A_BYTES, &tmA, a_land, (kb_begin + j) * DG_BK, 0);
      }
      ok = mbar_wait_warp(a_land, 0, abort_flag, p.status, kStatusWaitTimeoutEpilogue);
      if (ok) {
        for (int j = 0; j < kb_cnt; ++j) {
          uint32_t v[32];
          const uint8_t* tile = land + j * DG_A_BYTES + row * 128;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const uint4 x = *reinterpret_cast<const uint4*>(tile + ((e ^ (row & 7)) << 4));
            v[4 * e] = x.x; v[4 * e + 1] = x.y; v[4 * e + 2] = x.z; v[4 * e + 3] = x.w;
          }
          dg_tmem_st32(tmem_base + lane_sel + j * 32, v);
        }
        dg_tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_ready);
      }
    } else if (p.pdl) {
      pdl_wait();                                   // its stores below still follow the predecessor
    }
    if (stamp) p.debug[1] = globaltimer_ns();
    // The landing zone overlaps the receive and staging buffers: nobody may send to me before my rows
    // are out of it.  a_ready has all four warps' arrivals once that is true; peers learn it through
    // the first peers_free round below (tiles 0 and 1 are sent only after the receivers said so).
    if (work && ok) ok = mbar_wait_warp(a_ready, 0, abort_flag, p.status, kStatusWaitTimeoutEpilogue);
    if (ok && my_tiles > 0) {
      __syncwarp();
      if (lane < DG_S && lane != rank) {
#pragma unroll
        for (int b = 0; b < DG_NBUF; ++b) dg_arrive_remote(dg_mapa(smem_u32(&peers_free[b * 4 + q]), lane));
      }
    }
    // Software pipeline: iteration t sends the partials of tile t and then finishes tile t - (DG_NBUF - 1),
    // whose partials have been travelling in the meantime (a bulk copy between CTAs takes about 2 us).
    uint32_t own_hist[DG_NBUF - 1][8];       // my own partials of the tiles still in flight, oldest first
#pragma unroll
    for (int i = 0; i < DG_NBUF - 1; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) own_hist[i][e] = 0u;
    for (int t = 0; t < my_tiles + DG_NBUF - 1 && ok && my_tiles > 0; ++t) {
      uint32_t own[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) own[e] = 0u;
      if (t < my_tiles) {
        const int ab = t & 1;                          // accumulator of this tile
        const int xb = t % DG_NBUF;                    // its staging and receive buffer
        const int use = t / DG_NBUF;
        uint32_t r[DG_BN];
        if (kb_cnt > 0) {
          ok = mbar_wait_warp(&acc_full[ab], (t >> 1) & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue);
          if (!ok) break;
          tc_fence_after();
          const uint32_t taddr = tmem_base + lane_sel + DG_ACC_COL + ab * DG_BN;
          tmem_ld32(taddr, r);
          tmem_ld32(taddr + 32, r + 32);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[ab]);          // the accumulator may be overwritten
        } else {
#pragma unroll
          for (int e = 0; e < DG_BN; ++e) r[e] = 0u;
        }
        if (stamp && t < 14) p.debug[2 + 4 * t] = globaltimer_ns();
        // every peer has consumed what I sent into this buffer DG_NBUF tiles ago (for the first tiles: has
        // emptied its landing zone), which also means the copies out of my staging buffer are done
        ok = dg_wait_cluster_warp(&peers_free[xb * 4 + q], use & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue);
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(&red_full[xb * 4 + q], (DG_S - 1) * DG_CHUNK);   // arm my own receive barrier
        uint8_t* sbuf = stg + xb * DG_RED_BYTES;
#pragma unroll
        for (int d = 0; d < DG_S; ++d) {
          const int r0 = dg_run0<GLU>(d), r1 = dg_run1<GLU>(d);
          if (d == rank) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              own[e] = r[r0 + e];
              own[4 + e] = r[r1 + e];
            }
          } else {
            const int pi = d < rank ? d : d - 1;                          // staging chunk of peer d
            float4* ch = reinterpret_cast<float4*>(sbuf + (pi * 4 + q) * DG_CHUNK);
            ch[lane] = make_float4(__uint_as_float(r[r0]), __uint_as_float(r[r0 + 1]), __uint_as_float(r[r0 + 2]), __uint_as_float(r[r0 + 3]));
            ch[32 + lane] = make_float4(__uint_as_float(r[r1]), __uint_as_float(r[r1 + 1]), __uint_as_float(r[r1 + 2]), __uint_as_float(r[r1 + 3]));
          }
        }
        fence_async_smem();                            // my staging writes are visible to the copy engine ...
        __syncwarp();                                  // ... and so are those of the other lanes
        if (lane < DG_S && lane != rank) {             // lane d sends this warp's chunk to rank d
          const int d = lane;
          const int pi = d < rank ? d : d - 1;
          const int slot = rank < d ? rank : rank - 1;                    // the receiver's slots skip its own rank
          dg_bulk_to_peer(dg_mapa(smem_u32(red + xb * DG_RED_BYTES + (slot * 4 + q) * DG_CHUNK), d),
                          smem_u32(sbuf + (pi * 4 + q) * DG_CHUNK), DG_CHUNK, dg_mapa(smem_u32(&red_full[xb * 4 + q]), d));
        }
        if (stamp && t < 14) p.debug[3 + 4 * t] = globaltimer_ns();
      }
      if (t >= DG_NBUF - 1) {
        const int tp = t - (DG_NBUF - 1);
        const int xb = tp % DG_NBUF;
        const int use = tp / DG_NBUF;
        const int ni = c + tp * p.C;
        const uint8_t* rbuf = red + xb * DG_RED_BYTES;
        ok = dg_wait_cluster_warp(&red_full[xb * 4 + q], use & 1, abort_flag, p.status, kStatusWaitTimeoutEpilogue);
        if (!ok) break;
        if (stamp && tp < 14) p.debug[4 + 4 * tp] = globaltimer_ns();
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
        for (int src = 0; src < DG_S; ++src) {        // rank order, my own partial in its place
          if (src == rank) {
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += __uint_as_float(own_hist[0][e]);
          } else {
            const int slot = src < rank ? src : src - 1;
            const float4* ch = reinterpret_cast<const float4*>(rbuf + (slot * 4 + q) * DG_CHUNK);
            const float4 x0 = ch[lane];
            const float4 x1 = ch[32 + lane];
            acc[0] += x0.x; acc[1] += x0.y; acc[2] += x0.z; acc[3] += x0.w;
            acc[4] += x1.x; acc[5] += x1.y; acc[6] += x1.z; acc[7] += x1.w;
          }
        }
        __syncwarp();                                  // every lane has read its slots
        // this buffer may be refilled by the partials of tile tp + DG_NBUF
        if (tp + DG_NBUF < my_tiles && lane < DG_S && lane != rank) dg_arrive_remote(dg_mapa(smem_u32(&peers_free[xb * 4 + q]), lane));
        if (row < p.M) {
          if (PARTIAL) {
            float* op = p.partial + (static_cast<long long>(g) * p.M + row) * p.N + ni * DG_BN + rank * 8;
            reinterpret_cast<float4*>(op)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            reinterpret_cast<float4*>(op)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
          } else if (GLU) {
            float o4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float gate = acc[e], up = acc[4 + e];
              float a;
              if (p.glu_act == 1) {
                a = gate / (1.f + __expf(-gate));
              } else {
                const float th = tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate));
                a = 0.5f * gate * (1.f + th);
              }
              o4[e] = a * up;
            }
            __nv_bfloat16* op = p.out + static_cast<long long>(row) * p.ldo + ni * (DG_BN / 2) + (rank / 2) * 8 + (rank % 2) * 4;
            const __nv_bfloat162 h0 = __floats2bfloat162_rn(o4[0], o4[1]), h1 = __floats2bfloat162_rn(o4[2], o4[3]);
            uint2 v;
            v.x = *reinterpret_cast<const uint32_t*>(&h0);
            v.y = *reinterpret_cast<const uint32_t*>(&h1);
            *reinterpret_cast<uint2*>(op) = v;
          } else {
            const int col = ni * DG_BN + rank * 8;
            if (HAS_RES) {
              const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(row) * p.ldr + col);
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h[e]);
                acc[2 * e] += f.x;
                acc[2 * e + 1] += f.y;
              }
            }
            uint4 v;
            uint32_t* vp = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
              vp[e] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(p.out + static_cast<long long>(row) * p.ldo + col) = v;
          }
        }
        if (stamp && tp < 14) p.debug[5 + 4 * tp] = globaltimer_ns();
      }
#pragma unroll
      for (int i = 0; i + 1 < DG_NBUF - 1; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) own_hist[i][e] = own_hist[i + 1][e];
#pragma unroll
      for (int e = 0; e < 8; ++e) own_hist[DG_NBUF - 2][e] = own[e];
    }
    if (stamp) p.debug[58] = globaltimer_ns();
  }

  // ---- common exit: nobody leaves while a peer may still copy into, or signal, this CTA
  tc_fence_before();
  __syncthreads();
  dg_cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(DG_TMEM_COLS) : "memory");
  }
}

// out[r, c] = sum_g partial[g, r, c] (+ residual), summed in group order; 8 columns per thread
template <bool HAS_RES>
__global__ void decode_gemm_reduce_kernel(const float* __restrict__ partial, int G, int M, int N, __nv_bfloat16* __restrict__ out,
                                          long long ldo, const __nv_bfloat16* __restrict__ residual, long long ldr) {
  pdl_trigger();
  pdl_wait();
  const long long n8 = N / 8;
  const long long total = static_cast<long long>(M) * n8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / n8;
    const int col = static_cast<int>(i % n8) * 8;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int g = 0; g < G; ++g) {
      const float4* pp = reinterpret_cast<const float4*>(partial + (static_cast<long long>(g) * M + row) * N + col);
      const float4 x0 = pp[0], x1 = pp[1];
      acc[0] += x0.x; acc[1] += x0.y; acc[2] += x0.z; acc[3] += x0.w;
      acc[4] += x1.x; acc[5] += x1.y; acc[6] += x1.z; acc[7] += x1.w;
    }
    if (HAS_RES) {
      const uint4 rv = *reinterpret_cast<const uint4*>(residual + row * ldr + col);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    uint4 v;
    uint32_t* vp = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      vp[e] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(out + row * ldo + col) = v;
  }
}

template <bool GLU, bool HAS_RES, bool PARTIAL>
const char* launch_decode_gemm(const DecodeGemmArgs& a, DgParams p, const CUtensorMap& tmA, const CUtensorMap& tmB,
                               cudaStream_t stream) {
  auto kern = decode_gemm_kernel<GLU, HAS_RES, PARTIAL>;
  if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DG_SMEM) == cudaSuccess))
    return "decode_gemm: cannot reserve shared memory";
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(DG_THREADS);
  cfg.dynamicSmemBytes = DG_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = DG_S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // how many clusters of 8 the device can hold at once (GPC sizes decide), asked once per device
  static int max_clusters[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return "decode_gemm: device ordinal out of range";
  if (max_clusters[dev] == 0) {
    cfg.gridDim = dim3(DG_S * 16);
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) return "decode_gemm: cluster occupancy query failed";
    max_clusters[dev] = n;
  }
  int clusters = max_clusters[dev];
  if (a.max_clusters > 0 && a.max_clusters < clusters) clusters = a.max_clusters;
  p.C = clusters / p.G;
  if (p.C < 1) return "decode_gemm: fewer co-resident clusters than k groups";
  if (p.C > p.n_tiles) p.C = p.n_tiles;
  cfg.gridDim = dim3(p.G * p.C * DG_S);
  cfg.numAttrs = p.pdl ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p) != cudaSuccess) return "decode_gemm: launch failed";
  count_launch();
  return nullptr;
}

}  // namespace

bool decode_gemm_supported(int M, int N, int K, bool glu) {
  if (M < 1 || M > DG_BM || N < DG_BN || (N % DG_BN) || (K % 8)) return false;
  const int kb_total = (K + DG_BK - 1) / DG_BK;
  if (kb_total < DG_S) return false;                       // every rank of the cluster gets at least one k-block
  const int G = (kb_total + DG_S * DG_RES - 1) / (DG_S * DG_RES);
  if (G > 8) return false;
  if (glu && G > 1) return false;                          // the activation needs the complete sum
  const int kb_group = (kb_total + G - 1) / G;
  // the last group must not leave a rank of its cluster without work either
  const int last = kb_total - (G - 1) * kb_group;
  const int per = (kb_group + DG_S - 1) / DG_S;
  if (last < 1 || (last + per - 1) / per < 1) return false;
  return true;
}

int decode_gemm_groups(int K) {
  const int kb_total = (K + DG_BK - 1) / DG_BK;
  return (kb_total + DG_S * DG_RES - 1) / (DG_S * DG_RES);
}

const char* decode_gemm(const DecodeGemmArgs& a, cudaStream_t stream) {
  if (!decode_gemm_supported(a.M, a.N, a.K, a.glu_act != 0)) return "decode_gemm: unsupported shape";
  if ((a.lda % 8) || (a.ldb % 8) || (a.ldo % 8) || (a.residual && (a.ldr % 8)))
    return "decode_gemm: row strides must be multiples of 8 elements";
  if ((reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15) ||
      (reinterpret_cast<uintptr_t>(a.out) & 15) || (a.residual && (reinterpret_cast<uintptr_t>(a.residual) & 15)))
    return "decode_gemm: operands must be 16-byte aligned";
  if (a.glu_act && a.residual) return "decode_gemm: no residual with the GLU epilogue";
  DgParams p{};
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.kb_total = (a.K + DG_BK - 1) / DG_BK;
  p.G = decode_gemm_groups(a.K);
  p.kb_group = (p.kb_total + p.G - 1) / p.G;
  p.n_tiles = a.N / DG_BN;
  p.out = static_cast<__nv_bfloat16*>(a.out); p.ldo = a.ldo;
  p.residual = static_cast<const __nv_bfloat16*>(a.residual); p.ldr = a.ldr;
  p.partial = a.partial;
  p.glu_act = a.glu_act;
  p.pdl = a.pdl ? 1 : 0;
  p.status = a.status;
  if (p.G > 1 && !a.partial) return "decode_gemm: K needs k groups and no fp32 workspace was given";
  p.A = static_cast<const __nv_bfloat16*>(a.A); p.lda = a.lda;
  p.debug = a.debug;
  CUtensorMap tmA, tmB;
  if (!make_map_2d(&tmA, a.A, a.M, a.K, a.lda, DG_BM)) return "decode_gemm: tensor map for A failed";
  if (!make_map_2d(&tmB, a.B, a.N, a.K, a.ldb, DG_BN)) return "decode_gemm: tensor map for B failed";
  const char* err;
  if (p.G > 1) {
    err = launch_decode_gemm<false, false, true>(a, p, tmA, tmB, stream);
    if (err) return err;
    const long long total = static_cast<long long>(a.M) * (a.N / 8);
    const int blocks = static_cast<int>((total + 255) / 256);
    cudaError_t e;
    if (a.residual)
      e = launch_pdl(decode_gemm_reduce_kernel<true>, dim3(blocks), dim3(256), 0, stream, a.partial, p.G, a.M, a.N, p.out, p.ldo,
                     p.residual, p.ldr);
    else
      e = launch_pdl(decode_gemm_reduce_kernel<false>, dim3(blocks), dim3(256), 0, stream, a.partial, p.G, a.M, a.N, p.out, p.ldo,
                     p.residual, p.ldr);
    if (e != cudaSuccess) return "decode_gemm: reduce launch failed";
    count_launch();
    return nullptr;
  }
  if (a.glu_act) return launch_decode_gemm<true, false, false>(a, p, tmA, tmB, stream);
  if (a.residual) return launch_decode_gemm<false, true, false>(a, p, tmA, tmB, stream);
  return launch_decode_gemm<false, false, false>(a, p, tmA, tmB, stream);
}

}  // namespace ferrl
