// bf16 GEMM core for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T  (+ A2[M,K2] * B2[N,K2]^T) (+ R[M,N])
//
// * tcgen05.mma (cta_group::1, kind::f16, M=128, N=BN, K=16 per instruction) issued by one
//   elected thread; fp32 accumulators live in TMEM, two of them so the epilogue of tile i
//   overlaps the main loop of tile i+1.
// * operands are staged in shared memory by TMA (cp.async.bulk.tensor.2d, 128B swizzle,
//   no cluster multicast: this kernel runs inside multi-GPU jobs) through an
//   mbarrier-driven ring of STAGES buffers.
// * the optional second operand pair (A2, B2) is the LoRA side path: A2 = x*A_stack^T
//   ([M, n*r]) and B2 = s*B_blockdiag ([N, n*r]) are consumed as extra k-tiles of the same
//   accumulator, so the low-rank delta costs no extra pass over the output.
// * persistent: one CTA per SM walks a grouped-M raster so concurrently running CTAs share
//   A and B tiles in L2.
// * warp roles: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 =
//   epilogue (tcgen05.ld -> convert -> 16-byte global stores, optional residual add).
// * every mbarrier wait is bounded: on expiry the role records a status code in global
//   memory, raises a CTA-wide abort flag, and all roles fall through to the common exit
//   where TMEM is released.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api.h"
#include "../common.cuh"
#include "../symm/symm.cuh"

namespace ferrl {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // 2 s

struct GemmParams {
  int M, N, K, K2;
  void* out;            // bf16 or fp32, row stride ldo elements
  const __nv_bfloat16* residual;  // optional [M, ldr]
  long long ldo, ldr;
  int* status;          // device status word
  int group_m;
  int split_k;          // > 1: each tile covers a slice of the k-tiles and writes fp32 partials
  int kb_per_split;
  float* partial;       // [split_k, M, N] fp32 when split_k > 1
  // grouped (mixture-of-experts) mode: A rows are sorted by expert in 128-row aligned segments,
  // B is [E * N, K]; tile_expert[mi] names the expert of m tile mi, or -1 for an unused tile.
  const int* tile_expert;
  // Fused all-reduce for tensor-parallel row-parallel projections, active when ar_world > 1.
  // All NVLink traffic is posted stores.  Output tile t belongs to rank t % world:
  //   1. every rank's epilogue writes its bf16 partial of tile t into the owner's staging buffer,
  //      slot [t / world][rank], in a chunk-major layout (a warp store covers 512 contiguous bytes),
  //      then releases ready[t][rank] in the owner's flags;
  //   2. the owner waits for all ready flags, sums the slots in rank order (+ residual), writes the
  //      tile into its own `out` and into every peer's `ar_outbuf`, and releases done[t] everywhere;
  //   3. every rank copies the tiles it does not own from its local `ar_outbuf` into `out` as their
  //      done flags arrive, between its own tiles where it can and in a final sweep for the rest.
  int ar_world, ar_rank;
  PeerTable ar_stage, ar_outbuf, ar_flags;
  int ar_max_tiles;
  uint64_t ar_limit_ns;
  unsigned long long* ar_debug;   // optional [grid][16 tiles][4] globaltimer stamps of the exchange
  // In-switch variant (both non-null): `ar_stage` and `ar_outbuf` are bound to NVSwitch multicast objects and these
  // are their multicast addresses.  Every rank then stores its partial of tile t in its OWN staging copy, slot t;
  // the owner reads the sum of all copies with `multimem.ld_reduce` (the switch adds), and one `multimem.st` per
  // chunk puts the reduced tile into every rank's receive buffer.  Flags, epochs and the copy-out are unchanged.
  void* ar_mc_stage;
  void* ar_mc_outbuf;
  // Reduce-scatter form (ar_scatter != 0, M a multiple of ar_world x BM): the owner of a tile is the rank that keeps
  // its rows, step 2 ends with the store into the owner's `out` [M / ar_world, N], and step 3 does not exist.  Each
  // rank walks the row blocks starting with its successor's and ending with its own, so the peers' partials of a tile
  // are in place when its owner reaches it.  Nothing flows back to the senders tile by tile; instead every rank's last
  // CTA publishes fin[rank] = call number on all peers, and a rank waits for fin >= previous call on its peers before
  // its first push of a call (both forms do: a sender may otherwise run ahead into staging slots still being summed).
  int ar_scatter;
  // All-gather -> GEMM (ar_gather != 0, M a multiple of ar_world x BM, A packed): A is this rank's gather buffer, of
  // which the caller filled this rank's M / ar_world rows.  CTA 0 tells every peer that the rows are in place
  // (agr[rank] = call number); the communication warps pull the peers' rows, 128 rows x 256 columns per unit and unit
  // by unit over all CTAs, into the local buffer and count arrived[m tile] up; the TMA producer loads a tile of
  // foreign rows only once its count is complete.  The tile sequence starts with this rank's own rows and continues
  // with the successors' in the order the units are pulled.  The output is the plain [M, N] one of this rank.
  // The caller alternates between two gather buffers: a peer may rewrite its rows for the call after next only after
  // this rank has published that call's number, i.e. has finished pulling for this one.
  int ar_gather;
  PeerTable ag_src;
  // Launched as a programmatic dependent: the producer fills its ring with the weight (B) halves of
  // its first k-blocks, which no earlier kernel writes, before it waits for the stream predecessor;
  // only then does it fetch the activation (A) halves.  Everything else in the kernel is ordered
  // behind those loads by the pipeline's barriers.
  int pdl;
  // Gated-linear-unit epilogue (one-SM kernel, bf16 output, no k-split): the N rows of B come in groups
  // of 16, eight gate rows followed by the eight up rows of the same features, and the kernel writes
  // act(gate) * up, N / 2 columns per row.  1 = SiLU, 2 = tanh-GELU.
  int glu_act;
  // Language-model head without a logits tensor (one-SM kernel with 256-wide tiles and the two-SM kernel).
  // Every accumulator value is first turned into the scored logit z = softcap(x) / T.
  //   lp_mode 1: nothing is stored to `out`; per row and column tile the epilogue writes the running
  //              (max, sum exp(z - max)) to lp_ws[tile][row], and the z of the target column to lp_tl[row];
  //   lp_mode 2: `out` receives d z-loss / d x = lp_coef[row] * (exp(z - lp_lse[row]) - [col == target]) *
  //              dz/dx as bf16 (the caller multiplies by the weight again for the hidden-state gradient).
  // B may be a slice of the vocabulary: lp_col0 is the vocabulary index of its first row.
  int lp_mode;
  const long long* lp_targets;
  float lp_inv_t, lp_cap;
  long long lp_col0;
  float2* lp_ws;
  float* lp_tl;
  const float* lp_lse;
  const float* lp_coef;
  // RMSNorm folded around the projection (decode): with ss_in the accumulator rows are scaled by
  // rstd[row] = rsqrt(sum_t ss_in[t][row] * ss_inv_k + ss_eps) (the norm weight lives in B's columns);
  // with ss_out the epilogue writes, per output row, the sum of squares of the values it stored to
  // ss_out[part][row] (part = column tile, or column tile x cluster rank), summed by the consumer in
  // part order: no atomics, so the normalisation stays bit-reproducible.
  const float* ss_in; int ss_parts; long long ss_ld; float ss_inv_k, ss_eps;
  float* ss_out;
};

// flag layout inside each rank's flag buffer: ready[tile][kMaxRanks] then done[tile]
__device__ __forceinline__ uint32_t* ar_ready(const PeerTable& f, int rank_mem, int tile, int from) {
  return static_cast<uint32_t*>(f.ptr[rank_mem]) + static_cast<long long>(tile) * kMaxRanks + from;
}
__device__ __forceinline__ uint32_t* ar_done(const PeerTable& f, int rank_mem, int max_tiles, int tile) {
  return static_cast<uint32_t*>(f.ptr[rank_mem]) + static_cast<long long>(max_tiles) * kMaxRanks + tile;
}
__device__ __forceinline__ uint32_t* ar_fin(const PeerTable& f, int rank_mem, int max_tiles, int from) {
  return static_cast<uint32_t*>(f.ptr[rank_mem]) + static_cast<long long>(max_tiles) * (kMaxRanks + 1) + 2 + from;
}
__device__ __forceinline__ uint32_t* ar_agr(const PeerTable& f, int rank_mem, int max_tiles, int from) {
  return static_cast<uint32_t*>(f.ptr[rank_mem]) + static_cast<long long>(max_tiles) * (kMaxRanks + 1) + 2 + kMaxRanks + from;
}
constexpr int kMaxGatherMTiles = 1024;
constexpr int kGatherUnitCols = 256;
__device__ __forceinline__ uint32_t* ar_arrived(const PeerTable& f, int rank_mem, int max_tiles) {
  return static_cast<uint32_t*>(f.ptr[rank_mem]) + static_cast<long long>(max_tiles) * (kMaxRanks + 1) + 2 + 2 * kMaxRanks;
}
__device__ __forceinline__ bool flag_reached(const uint32_t* flag, uint32_t epoch) {
  return static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0;   // epochs only grow; tolerates wrap-around
}

// Bounded spin on a flag word in local memory; one thread calls it.
__device__ __forceinline__ bool ar_wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t limit_ns, int* status) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!flag_reached(flag, epoch)) {
    if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > limit_ns) {
      atomicCAS(status, kStatusOk, kStatusPeerWaitTimeout);
      return false;
    }
  }
  return true;
}

// Bounded spin until a device-scope counter in local memory has reached `want`; one thread calls it.
__device__ __forceinline__ bool ar_wait_count(const uint32_t* ctr, uint32_t want, uint64_t limit_ns, int* status) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= want) return true;
    if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > limit_ns) {
      atomicCAS(status, kStatusOk, kStatusPeerWaitTimeout);
      return false;
    }
  }
}

__device__ __forceinline__ uint4 pack8(const float* a) {
  uint4 o;
  uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * e], a[2 * e + 1]);
    op[e] = *reinterpret_cast<uint32_t*>(&h);
  }
  return o;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st16(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void add8(float* a, const uint4& x) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float2 f = __bfloat1622float2(h[e]);
    a[2 * e] += f.x;
    a[2 * e + 1] += f.y;
  }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. Returns false when the CTA is aborting or the limit expired (and then
// records `code`).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code, uint64_t limit_ns = WAIT_LIMIT_NS) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        atomicCAS(status, kStatusOk, code);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// K-major, 128B-swizzled operand tile: rows are 128 bytes, 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);   // start address
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
  return d;
}

__host__ __device__ constexpr uint32_t make_idesc(int n) {
  return (1u << 4)                        // D format F32
         | (1u << 7)                      // A format BF16
         | (1u << 10)                     // B format BF16
         | (static_cast<uint32_t>(n >> 3) << 17)
         | (static_cast<uint32_t>(BM >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- log-prob epilogue (see GemmParams::lp_mode): per-thread state of one output row
struct LpRow {
  float m, s, tl, lse, coef;
  long long tgt;       // target column relative to this call's first column (may be out of range)
  bool hit;
};
__device__ __forceinline__ void lp_begin(const GemmParams& p, int row, bool row_ok, LpRow& st) {
  st.m = -INFINITY; st.s = 0.f; st.tl = 0.f; st.hit = false; st.lse = 0.f; st.coef = 0.f; st.tgt = -1;
  if (!row_ok) return;
  st.tgt = p.lp_targets[row] - p.lp_col0;
  if (p.lp_mode == 2) {
    st.lse = p.lp_lse[row];
    st.coef = p.lp_coef[row];
  }
}
// r holds 32 accumulator columns starting at column `col`; the first `ncols` are inside the matrix.
__device__ __forceinline__ void lp_chunk(const GemmParams& p, uint32_t* r, int col, int ncols, LpRow& st) {
  const float cap = p.lp_cap, inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  if (p.lp_mode == 1) {
    float cm = -INFINITY;
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      float z = __uint_as_float(r[e]);
      if (cap > 0.f) z = cap * tanhf(z * inv_cap);
      z *= p.lp_inv_t;
      if (e >= ncols) z = -INFINITY;
      if (col + e == st.tgt) { st.tl = z; st.hit = true; }
      r[e] = __float_as_uint(z);
      cm = fmaxf(cm, z);
    }
    const float nm = fmaxf(st.m, cm);
    float add = 0.f;
#pragma unroll
    for (int e = 0; e < 32; ++e) add += __expf(__uint_as_float(r[e]) - nm);
    st.s = st.s * __expf(st.m - nm) + add;
    st.m = nm;
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const float x = __uint_as_float(r[e]);
      float z = x, dz = p.lp_inv_t;
      if (cap > 0.f) {
        const float t = tanhf(x * inv_cap);
        z = cap * t;
        dz *= 1.f - t * t;
      }
      z *= p.lp_inv_t;
      const float pr = __expf(z - st.lse) - ((col + e == st.tgt) ? 1.f : 0.f);
      r[e] = __float_as_uint(st.coef * pr * dz);
    }
  }
}
__device__ __forceinline__ void lp_end(const GemmParams& p, int row, bool row_ok, int ni, const LpRow& st) {
  if (p.lp_mode != 1 || !row_ok) return;
  p.lp_ws[static_cast<long long>(ni) * p.M + row] = make_float2(st.m, st.s);
  if (st.hit) p.lp_tl[row] = st.tl;
}

template <int BN> struct Cfg {
  static constexpr int STAGE_BYTES = (BM + BN) * BK * 2;
  static constexpr int STAGES = (BN >= 256) ? 4 : (BN > 128 ? 5 : (BN >= 128 ? 6 : 8));
  static constexpr int TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void tile_coords_mn(int tile, int m_tiles, int n_tiles, int group_m, int& mi, int& ni) {
  int per_group = group_m * n_tiles;
  int g = tile / per_group;
  int first_m = g * group_m;
  int gsz = min(group_m, m_tiles - first_m);
  int in = tile - g * per_group;
  mi = first_m + in % gsz;
  ni = in / gsz;
}

// tile index -> (k-split, m tile, n tile); splits of one output tile are adjacent so they share L2 lines
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int group_m, int split_k, int& ks,
                                            int& mi, int& ni) {
  ks = tile % split_k;
  tile_coords_mn(tile / split_k, m_tiles, n_tiles, group_m, mi, ni);
}

// Tile order of the fused collective forms.  All-reduce: the plain order.  Reduce-scatter (1): row block by row block,
// the successor's first and this rank's own last (the plain order inside a block).  All-gather (2): this rank's own
// block first, then the successors'.
template <bool AR>
__device__ __forceinline__ void tile_coords_ar(int ar_scatter, int ar_rank, int ar_world, int tile, int m_tiles, int n_tiles,
                                               int group_m, int split_k, int& ks, int& mi, int& ni) {
  if (AR && ar_scatter) {
    const int mt_per = m_tiles / ar_world, per = mt_per * n_tiles;
    const int blk = tile / per;
    int owner = ar_rank + blk + (ar_scatter == 2 ? 0 : 1);      // 2: gather order, own rows first
    if (owner >= ar_world) owner -= ar_world;
    int ml;
    tile_coords_mn(tile - blk * per, mt_per, n_tiles, group_m, ml, ni);
    mi = owner * mt_per + ml;
    ks = 0;
  } else {
    tile_coords(tile, m_tiles, n_tiles, group_m, split_k, ks, mi, ni);
  }
}
// owner of an output tile and the first staging slot of its group of ar_world slots in the owner's buffer
__device__ __forceinline__ void ar_owner_slot(int ar_scatter, int ar_world, int m_tiles, int n_tiles, int mi, int ni,
                                              int& owner, long long& slot0) {
  if (ar_scatter) {
    const int mt_per = m_tiles / ar_world;
    owner = mi / mt_per;
    slot0 = (static_cast<long long>(mi - owner * mt_per) * n_tiles + ni) * ar_world;
  } else {
    const int out_tile = mi * n_tiles + ni;
    owner = out_tile % ar_world;
    slot0 = static_cast<long long>(out_tile / ar_world) * ar_world;
  }
}

// OUT_F32: write fp32 instead of bf16.  HAS_RES: add a bf16 residual tile before the store.
// AR: fused all-reduce mode (compiled separately so the plain kernel carries none of its registers).
// rstd of one row from the partial sums of squares its producer wrote (summed in part order, 16 loads in
// flight at a time: the epilogue threads call this while the main loop is still running)
__device__ __forceinline__ float row_rstd(const float* __restrict__ ss, int parts, long long ld, int row, float inv_k, float eps) {
  float sacc = 0.f;
  for (int t0 = 0; t0 < parts; t0 += 16) {
    float v[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) v[k] = (t0 + k < parts) ? ss[(t0 + k) * ld + row] : 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) sacc += v[k];
  }
  return rsqrtf(sacc * inv_k + eps);
}

template <int BN, bool OUT_F32, bool HAS_RES, bool AR>
__global__ void __launch_bounds__(AR ? NUM_THREADS + 128 : NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2, GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES]
  uint64_t* empty = bars + C::STAGES;       // [STAGES]
  uint64_t* acc_full = bars + 2 * C::STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;          // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* epi_bar = acc_empty + 3;           // epilogue-group barrier (4 warps) of the all-reduce mode
  volatile int* pull_ready = reinterpret_cast<volatile int*>(acc_empty + 4);
  uint64_t* comm_bar = acc_empty + 5;          // communication-group barrier (4 warps), all-reduce mode
  volatile int* drained = reinterpret_cast<volatile int*>(acc_empty + 6);   // tiles whose partial has left TMEM
  // a peer may enter the kernel later than this rank: every wait of the all-reduce mode allows for that skew
  const uint64_t wait_limit = AR ? WAIT_LIMIT_NS + p.ar_limit_ns : WAIT_LIMIT_NS;
  // The call number lives in this rank's flag buffer and is advanced by the kernel itself (last CTA
  // out), so a captured CUDA graph replays with fresh flag values; ranks call in lockstep, so their
  // counters agree.
  uint32_t* ar_epoch_word = nullptr;
  uint32_t ar_epoch = 0;
  if (AR) {
    ar_epoch_word = static_cast<uint32_t*>(p.ar_flags.ptr[p.ar_rank]) + static_cast<long long>(p.ar_max_tiles) * (kMaxRanks + 1);
    ar_epoch = *reinterpret_cast<volatile uint32_t*>(ar_epoch_word) + 1;
    if (p.ar_gather && blockIdx.x == 0 && threadIdx.x == 0)     // this rank's rows were written before the launch
      for (int q2 = 0; q2 < p.ar_world; ++q2)
        if (q2 != p.ar_rank) st_release_sys(ar_agr(p.ar_flags, q2, p.ar_max_tiles, p.ar_rank), ar_epoch);
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles * p.split_k;
  const int kb1 = (p.K + BK - 1) / BK;
  const int kb2 = (p.K2 + BK - 1) / BK;
  const int kb_total = kb1 + kb2;
  if (threadIdx.x == 0) pdl_trigger();   // a dependent kernel may start its own prologue now

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    mbar_init(epi_bar, 4);
    mbar_init(comm_bar, 4);
    *drained = 0;
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int pre = 0;          // k-blocks of the first tile whose loads were issued around the dependency wait
      if (p.pdl && static_cast<int>(blockIdx.x) < total_tiles) {
        int ks, mi, ni;
        tile_coords_ar<AR>(p.ar_gather ? 2 : p.ar_scatter, p.ar_rank, p.ar_world, blockIdx.x, m_tiles, n_tiles, p.group_m, p.split_k, ks, mi, ni);
        const int kb_begin = ks * p.kb_per_split, kb_end = min(kb_total, kb_begin + p.kb_per_split);
        pre = min(C::STAGES, kb_end - kb_begin);
        for (int i = 0; i < pre; ++i) {           // first pass over the ring: every stage is free
          const int kb = kb_begin + i;
          uint8_t* sb = smem + i * C::STAGE_BYTES + BM * BK * 2;
          mbar_expect_tx(&full[i], C::STAGE_BYTES);
          if (kb < kb1) tma_load_2d(sb, &tmB, &full[i], kb * BK, ni * BN);
          else tma_load_2d(sb, &tmB2, &full[i], (kb - kb1) * BK, ni * BN);
        }
        pdl_wait();
        for (int i = 0; i < pre; ++i) {
          const int kb = kb_begin + i;
          uint8_t* sa = smem + i * C::STAGE_BYTES;
          if (kb < kb1) tma_load_2d(sa, &tmA, &full[i], kb * BK, mi * BM);
          else tma_load_2d(sa, &tmA2, &full[i], (kb - kb1) * BK, mi * BM);
        }
        if (pre == C::STAGES) phase = 1; else stage = pre;
      }
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int ks, mi, ni;
        tile_coords_ar<AR>(p.ar_gather ? 2 : p.ar_scatter, p.ar_rank, p.ar_world, tile, m_tiles, n_tiles, p.group_m, p.split_k, ks, mi, ni);
        int b_row0 = ni * BN;
        if (p.tile_expert) {
          const int e = p.tile_expert[mi];
          if (e < 0) continue;
          b_row0 += e * p.N;
        }
        int kb_begin = ks * p.kb_per_split;
        const int kb_end = min(kb_total, kb_begin + p.kb_per_split);
        if (tile == static_cast<int>(blockIdx.x)) kb_begin += pre;
        if (AR && p.ar_gather && mi / (m_tiles / p.ar_world) != p.ar_rank) {
          // rows of a peer: all their column units must have landed in the local buffer (generic-proxy stores of
          // other CTAs, read here through the async proxy)
          const uint32_t units = (p.K + kGatherUnitCols - 1) / kGatherUnitCols;
          if (!ar_wait_count(ar_arrived(p.ar_flags, p.ar_rank, p.ar_max_tiles) + mi, units, wait_limit, p.status)) {
            *abort_flag = 1;
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer, wait_limit)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::STAGE_BYTES;
          uint8_t* sb = sa + BM * BK * 2;
          mbar_expect_tx(&full[stage], C::STAGE_BYTES);
          if (kb < kb1) {
            tma_load_2d(sa, &tmA, &full[stage], kb * BK, mi * BM);
            tma_load_2d(sb, &tmB, &full[stage], kb * BK, b_row0);
          } else {
            tma_load_2d(sa, &tmA2, &full[stage], (kb - kb1) * BK, mi * BM);
            tma_load_2d(sb, &tmB2, &full[stage], (kb - kb1) * BK, b_row0);
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // give copies already in flight time to land before the CTA's shared memory goes away
        for (int i = 0; i < 64; ++i) __nanosleep(10000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (p.tile_expert) {
          int ks_, mi_, ni_;
          tile_coords_ar<AR>(p.ar_gather ? 2 : p.ar_scatter, p.ar_rank, p.ar_world, tile, m_tiles, n_tiles, p.group_m, p.split_k, ks_, mi_, ni_);
          if (p.tile_expert[mi_] < 0) continue;
        }
        const int acc = (it++) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase[acc] ^ 1, abort_flag, p.status, kStatusWaitTimeoutMma, wait_limit)) break;
        acc_phase[acc] ^= 1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int ks = tile % p.split_k;
        const int kb_begin = ks * p.kb_per_split, kb_end = min(kb_total, kb_begin + p.kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, kStatusWaitTimeoutMma, wait_limit)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + BM * BK * 2;
          const uint64_t da = make_smem_desc(sa);
          const uint64_t db = make_smem_desc(sb);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advance 32 bytes (16 bf16) inside the 128-byte swizzle row: +2 in 16-byte units
            umma(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[stage]);  // frees the smem stage when these MMAs retire
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[acc]);
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue warps
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t acc_phase[2] = {0, 0};
    int it = 0;
    // ---- all-reduce mode state
    const int et = threadIdx.x - 64;              // 0..127 within the epilogue group
    uint32_t epi_phase = 0;
    auto epi_sync = [&]() -> bool {               // bounded barrier over the 4 epilogue warps
      __syncwarp();
      if (lane == 0) mbar_arrive(epi_bar);
      const bool ok = mbar_wait(epi_bar, epi_phase, abort_flag, p.status, kStatusWaitTimeoutEpilogue, wait_limit);
      epi_phase ^= 1;
      return ok && !*abort_flag;
    };
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      int ks, mi, ni;
      tile_coords_ar<AR>(p.ar_gather ? 2 : p.ar_scatter, p.ar_rank, p.ar_world, tile, m_tiles, n_tiles, p.group_m, p.split_k, ks, mi, ni);
      if (p.tile_expert && p.tile_expert[mi] < 0) continue;
      const int row = mi * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      float rstd = 1.f, ssq = 0.f;
      if (p.ss_in) {
        // gathered while the main loop runs; the statistics come from the stream predecessor, and this
        // thread is not ordered behind the producer warp's dependency wait yet
        if (p.pdl) pdl_wait();
        if (row_ok) rstd = row_rstd(p.ss_in, p.ss_parts, p.ss_ld, row, p.ss_inv_k, p.ss_eps);
      }
      const int acc = (it++) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase[acc], abort_flag, p.status, kStatusWaitTimeoutEpilogue, wait_limit)) break;
      acc_phase[acc] ^= 1;
      tc_fence_after();
      const int out_tile = mi * n_tiles + ni;
      __nv_bfloat16* ar_slot = nullptr;
      int owner = 0;
      if (AR && !p.ar_gather) {
        long long slot0;
        ar_owner_slot(p.ar_scatter, p.ar_world, m_tiles, n_tiles, mi, ni, owner, slot0);
        ar_slot = p.ar_mc_stage
                      ? static_cast<__nv_bfloat16*>(p.ar_stage.ptr[p.ar_rank]) + static_cast<long long>(out_tile) * (BM * BN)
                      : static_cast<__nv_bfloat16*>(p.ar_stage.ptr[owner]) + (slot0 + p.ar_rank) * (BM * BN);
        if (it == 1) {
          // first push of this call: every peer must have left the previous call, or its staging slots may still be read
          if (et == 0) {
            bool ok = true;
            for (int q2 = 0; q2 < p.ar_world && ok; ++q2)
              if (q2 != p.ar_rank)
                ok = ar_wait_flag(ar_fin(p.ar_flags, p.ar_rank, p.ar_max_tiles, q2), ar_epoch - 1, p.ar_limit_ns, p.status);
            if (!ok) *abort_flag = 1;
          }
          if (!epi_sync()) break;
        }
      }
      LpRow lp;
      if (p.lp_mode) lp_begin(p, row, row_ok, lp);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c, r);
        tmem_ld_wait();
        const int col = ni * BN + c;
        if (p.lp_mode) {
          if (!(row_ok && col < p.N)) continue;
          lp_chunk(p, r, col, min(min(32, BN - c), p.N - col), lp);
          if (p.lp_mode == 1) continue;
        }
        if (p.split_k > 1) {
          // fp32 partial of this k-slice; residual and the output cast happen in the reduce kernel
          if (row_ok && col < p.N) {
            const int ncols = min(min(32, BN - c), p.N - col);
            float* op = p.partial + (static_cast<long long>(ks) * p.M + row) * p.N + col;
            if (ncols == 32 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                reinterpret_cast<uint4*>(op)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            } else {
              for (int e = 0; e < ncols; ++e) op[e] = __uint_as_float(r[e]);
            }
          }
          continue;
        }
        if (AR && !p.ar_gather) {
          // bf16 partial of this rank, pushed into the tile owner's staging slot; rows past M hold the
          // zero fill of the TMA load, so no bounds test is needed inside the slot
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float f8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f8[e] = __uint_as_float(r[v * 8 + e]);
            reinterpret_cast<uint4*>(ar_slot)[(c / 8 + v) * BM + q * 32 + lane] = pack8(f8);
          }
          continue;
        }
        if (row_ok && col < p.N) {
          const int ncols = min(min(32, BN - c), p.N - col);
          if (p.ss_in) {
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * rstd);
          }
          if (HAS_RES) {
            const __nv_bfloat16* rp = p.residual + static_cast<long long>(row) * p.ldr + col;
            if (ncols == 32 && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 x = reinterpret_cast<const uint4*>(rp)[v];
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  float2 f = __bfloat1622float2(h[e]);
                  r[v * 8 + 2 * e] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * e]) + f.x);
                  r[v * 8 + 2 * e + 1] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * e + 1]) + f.y);
                }
              }
            } else {
              for (int e = 0; e < ncols; ++e)
                r[e] = __float_as_uint(__uint_as_float(r[e]) + __bfloat162float(rp[e]));
            }
          }
          if (OUT_F32) {
            float* op = reinterpret_cast<float*>(p.out) + static_cast<long long>(row) * p.ldo + col;
            if (ncols == 32 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                reinterpret_cast<uint4*>(op)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            } else {
              for (int e = 0; e < ncols; ++e) op[e] = __uint_as_float(r[e]);
            }
          } else if (p.glu_act) {
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldo + (col >> 1);
#pragma unroll
            for (int g16 = 0; g16 < 2; ++g16) {
              if (g16 * 16 < ncols) {
                float o8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float gate = __uint_as_float(r[g16 * 16 + e]), up = __uint_as_float(r[g16 * 16 + 8 + e]);
                  float a;
                  if (p.glu_act == 1) {
                    a = gate / (1.f + __expf(-gate));
                  } else {
                    const float t = tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate));
                    a = 0.5f * gate * (1.f + t);
                  }
                  o8[e] = a * up;
                }
                *reinterpret_cast<uint4*>(op + g16 * 8) = pack8(o8);
              }
            }
          } else {
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldo + col;
            if (ncols == 32 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 x;
                uint32_t* xp = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * e]),
                                                          __uint_as_float(r[v * 8 + 2 * e + 1]));
                  xp[e] = *reinterpret_cast<uint32_t*>(&h);
                  if (p.ss_out) {
                    const float2 hf = __bfloat1622float2(h);
                    ssq += hf.x * hf.x + hf.y * hf.y;
                  }
                }
                reinterpret_cast<uint4*>(op)[v] = x;
              }
            } else {
              for (int e = 0; e < ncols; ++e) {
                const __nv_bfloat16 hb = __float2bfloat16_rn(__uint_as_float(r[e]));
                op[e] = hb;
                if (p.ss_out) ssq += __bfloat162float(hb) * __bfloat162float(hb);
              }
            }
          }
        }
      }
      if (p.ss_out && row_ok) p.ss_out[ni * p.ss_ld + row] = ssq;
      if (p.lp_mode) lp_end(p, row, row_ok, ni, lp);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);   // TMEM is free again: the MMA warp moves on while we talk to peers
      if (AR && !p.ar_gather) {
        // The exchange itself belongs to the communication warps below; here the tile is only
        // announced.  One system-scope release per tile, by one thread: the barrier orders the other
        // threads' stores before it.  A tile this rank owns is announced through shared memory.
        if (p.ar_debug && et == 0) p.ar_debug[(blockIdx.x * 16 + min(it - 1, 15)) * 4 + 0] = globaltimer_ns();
        if (!epi_sync()) break;
        if (et == 0) {
          // in-switch variant: the partial sits in local memory and is read through the switch.  For a peer's
          // tile the system-scope release below orders it; for a tile of this rank the hand-over to the
          // communication warps is only CTA-scoped, so the partial is made visible device-wide first
          if (p.ar_mc_stage && owner == p.ar_rank) __threadfence();
          if (owner != p.ar_rank) st_release_sys(ar_ready(p.ar_flags, owner, out_tile, p.ar_rank), ar_epoch);
          asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(const_cast<int*>(drained))), "r"(it) : "memory");
        }
        if (p.ar_debug && et == 0) p.ar_debug[(blockIdx.x * 16 + min(it - 1, 15)) * 4 + 1] = globaltimer_ns();
      }
    }
  } else if (AR) {
    // ------------------------------------------------------------ communication warps (all-reduce mode only)
    // They walk the same tile sequence as the epilogue, one or more tiles behind it, and never touch
    // TMEM: waiting for peers, the owner's reduction, the pushes and the copies of the peers' tiles
    // run beside the tensor cores instead of holding up the accumulator ring.
    const int ct = threadIdx.x - 192;             // 0..127
    if (p.ar_gather) {
      // ---- all-gather -> GEMM: pull the peers' rows of A into the local buffer, in the order the tiles need them
      const int mt_per = m_tiles / p.ar_world;
      const int kch = (p.K + kGatherUnitCols - 1) / kGatherUnitCols;
      const int units = (p.ar_world - 1) * mt_per * kch;
      uint32_t* arrived = ar_arrived(p.ar_flags, p.ar_rank, p.ar_max_tiles);
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.ag_src.ptr[p.ar_rank]);
      uint32_t gphase = 0, seen = 0;
      auto gsync = [&]() -> bool {
        __syncwarp();
        if (lane == 0) mbar_arrive(comm_bar);
        const bool ok = mbar_wait(comm_bar, gphase, abort_flag, p.status, kStatusWaitTimeoutEpilogue, wait_limit);
        gphase ^= 1;
        return ok && !*abort_flag;
      };
      for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int kc = u % kch, mt = (u / kch) % mt_per, blk = u / (kch * mt_per) + 1;
        int src = p.ar_rank + blk;
        if (src >= p.ar_world) src -= p.ar_world;
        if (ct == 0 && !((seen >> src) & 1u) &&
            !ar_wait_flag(ar_agr(p.ar_flags, p.ar_rank, p.ar_max_tiles, src), ar_epoch, wait_limit, p.status))
          *abort_flag = 1;
        seen |= 1u << src;
        if (!gsync()) break;
        const int mi = src * mt_per + mt;
        const int c0 = kc * kGatherUnitCols;
        const int nc8 = min(kGatherUnitCols, p.K - c0) >> 3;          // 16-byte pieces per row of this unit
        const int total = BM * nc8;
        const __nv_bfloat16* from = static_cast<const __nv_bfloat16*>(p.ag_src.ptr[src]);
        constexpr int UG = 8;
        for (int i0 = ct; i0 < total; i0 += 128 * UG) {
          uint4 x[UG];
          long long off[UG];
#pragma unroll
          for (int v = 0; v < UG; ++v) {
            const int i = i0 + v * 128;
            off[v] = -1;
            if (i < total) {
              off[v] = (static_cast<long long>(mi) * BM + i / nc8) * p.K + c0 + (i % nc8) * 8;
              x[v] = *reinterpret_cast<const uint4*>(from + off[v]);
            }
          }
#pragma unroll
          for (int v = 0; v < UG; ++v)
            if (off[v] >= 0) *reinterpret_cast<uint4*>(dst + off[v]) = x[v];
        }
        __threadfence();
        asm volatile("fence.proxy.async.global;" ::: "memory");
        if (!gsync()) break;
        if (ct == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(arrived + mi) : "memory");
      }
    } else {
    constexpr int CPR = BN / 8;
    const int out_tiles = m_tiles * n_tiles;
    auto peer_tile = [&](int u) -> int {
      const int g = u / (p.ar_world - 1), pos = u % (p.ar_world - 1);
      return g * p.ar_world + (pos < p.ar_rank ? pos : pos + 1);
    };
    int pull_u = blockIdx.x;
    uint32_t comm_phase = 0;
    auto comm_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(comm_bar);
      const bool ok = mbar_wait(comm_bar, comm_phase, abort_flag, p.status, kStatusWaitTimeoutEpilogue, wait_limit);
      comm_phase ^= 1;
      return ok && !*abort_flag;
    };
    auto copy_tile = [&](int t) {                 // local ar_outbuf -> out, one tile, 8 chunks in flight per thread
      const int tmi = t / n_tiles, tni = t % n_tiles;
      const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.ar_outbuf.ptr[p.ar_rank]);
      constexpr int UC = 8;
      for (int i0 = ct; i0 < BM * CPR; i0 += 128 * UC) {
        uint4 x[UC];
        long long so[UC];
        bool ok[UC];
#pragma unroll
        for (int u = 0; u < UC; ++u) {
          const int i = i0 + u * 128;
          const int rr = tmi * BM + i / CPR, cc = tni * BN + (i % CPR) * 8;
          ok[u] = i < BM * CPR && rr < p.M && cc < p.N;
          so[u] = static_cast<long long>(rr) * p.ldo + cc;
          if (ok[u]) x[u] = *reinterpret_cast<const uint4*>(src + static_cast<long long>(rr) * p.N + cc);
        }
#pragma unroll
        for (int u = 0; u < UC; ++u)
          if (ok[u]) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + so[u]) = x[u];
      }
    };
    int it = 0;
    bool live_c = true;
    for (int tile = blockIdx.x; tile < total_tiles && live_c; tile += gridDim.x) {
      int ks, mi, ni;
      tile_coords_ar<AR>(p.ar_gather ? 2 : p.ar_scatter, p.ar_rank, p.ar_world, tile, m_tiles, n_tiles, p.group_m, p.split_k, ks, mi, ni);
      ++it;
      const int out_tile = mi * n_tiles + ni;
      int owner;
      long long slot_first;
      ar_owner_slot(p.ar_scatter, p.ar_world, m_tiles, n_tiles, mi, ni, owner, slot_first);
      const int row_shift = p.ar_scatter ? p.ar_rank * (m_tiles / p.ar_world) * BM : 0;   // `out` holds this rank's rows only
      if (owner == p.ar_rank) {
        if (ct == 0) {
          // my own partial is in place once the epilogue has drained tile number `it`
          const uint64_t t0 = globaltimer_ns();
          uint32_t spins = 0;
          bool ok = true;
          while (*drained < it) {
            if ((++spins & 0xff) == 0 && (*abort_flag || globaltimer_ns() - t0 > wait_limit)) { ok = false; break; }
          }
          asm volatile("fence.acq_rel.cta;" ::: "memory");
          for (int q2 = 0; q2 < p.ar_world && ok; ++q2)
            if (q2 != p.ar_rank)
              ok = ar_wait_flag(ar_ready(p.ar_flags, p.ar_rank, out_tile, q2), ar_epoch, p.ar_limit_ns, p.status);
          if (!ok) *abort_flag = 1;
        }
        if (!comm_sync()) break;
        const uint4* slot0 = reinterpret_cast<const uint4*>(
            static_cast<const __nv_bfloat16*>(p.ar_stage.ptr[p.ar_rank]) + slot_first * (BM * BN));
        // U elements per round; the residual and WCH slots of each are requested before the first add
        // (the loop is bound by the latency of these loads, so what counts is how many are in flight)
        constexpr int U = 4, WCH = 4;
        if (p.ar_mc_stage) {
          // the switch forms the sum over all ranks' copies of slot `out_tile`; U requests in flight per thread
          // (eight per thread measured the same: the rate of the in-switch reduction, not this loop's depth, is the limit)
          const uint4* mc_tile = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.ar_mc_stage) +
                                                                static_cast<long long>(out_tile) * (BM * BN));
          __nv_bfloat16* mc_out = static_cast<__nv_bfloat16*>(p.ar_mc_outbuf);
          for (int i0 = ct; i0 < BM * CPR; i0 += 128 * U) {
            uint4 x[U], resv[U];
            bool live[U];
            int rr_[U], cc_[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int i = i0 + u * 128;
              const int rt = i / CPR, ch = i % CPR;
              rr_[u] = mi * BM + rt;
              cc_[u] = ni * BN + ch * 8;
              live[u] = i < BM * CPR && rr_[u] < p.M && cc_[u] < p.N;
              resv[u] = make_uint4(0u, 0u, 0u, 0u);
              x[u] = make_uint4(0u, 0u, 0u, 0u);
              if (live[u]) {
                x[u] = multimem_ld_reduce_bf16(mc_tile + ch * BM + rt);
                if (HAS_RES) resv[u] = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(rr_[u]) * p.ldr + cc_[u]);
              }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
              if (!live[u]) continue;
              uint4 o = x[u];
              if (HAS_RES) {
                float a8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) a8[e] = 0.f;
                add8(a8, x[u]);
                add8(a8, resv[u]);
                o = pack8(a8);
              }
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(rr_[u]) * p.ldo + cc_[u]) = o;
              multimem_st16(mc_out + static_cast<long long>(rr_[u]) * p.N + cc_[u], o);     // every rank's receive buffer at once
            }
          }
        } else
        for (int i0 = ct; i0 < BM * CPR; i0 += 128 * U) {
          float a8[U][8];
          bool live[U];
          int rr_[U], cc_[U];
          uint4 resv[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int i = i0 + u * 128;
            const int rt = i / CPR, ch = i % CPR;
            rr_[u] = mi * BM + rt;
            cc_[u] = ni * BN + ch * 8;
            live[u] = i < BM * CPR && rr_[u] < p.M && cc_[u] < p.N;
            resv[u] = make_uint4(0u, 0u, 0u, 0u);
            if (HAS_RES && live[u]) resv[u] = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(rr_[u]) * p.ldr + cc_[u]);
#pragma unroll
            for (int e = 0; e < 8; ++e) a8[u][e] = 0.f;
          }
          for (int w0 = 0; w0 < p.ar_world; w0 += WCH) {
            uint4 x[U][WCH];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int i = i0 + u * 128;
              const int rt = i / CPR, ch = i % CPR;
#pragma unroll
              for (int w = 0; w < WCH; ++w)
                if (live[u] && w0 + w < p.ar_world) x[u][w] = slot0[(w0 + w) * (BM * CPR) + ch * BM + rt];
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
              for (int w = 0; w < WCH; ++w)
                if (live[u] && w0 + w < p.ar_world) add8(a8[u], x[u][w]);      // rank order
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (!live[u]) continue;
            if (HAS_RES) add8(a8[u], resv[u]);
            const uint4 o = pack8(a8[u]);
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(rr_[u] - row_shift) * p.ldo + cc_[u]) = o;
            if (p.ar_scatter) continue;
            const long long off = static_cast<long long>(rr_[u]) * p.N + cc_[u];
            for (int q2 = 0; q2 < p.ar_world; ++q2)
              if (q2 != p.ar_rank) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.ar_outbuf.ptr[q2]) + off) = o;
          }
        }
        if (p.ar_debug && ct == 0) p.ar_debug[(blockIdx.x * 16 + min(it - 1, 15)) * 4 + 2] = globaltimer_ns();
        if (p.ar_scatter) continue;
        if (!comm_sync()) break;
        if (ct == 0) {
          // the release store orders this thread's view (which includes the other threads' pushes,
          // through the barrier above) before the flag; a separate sequentially-consistent system
          // fence in front of it cost 60 us per tile while the epilogue warps were pushing too
          for (int q2 = 0; q2 < p.ar_world; ++q2)
            if (q2 != p.ar_rank) st_release_sys(ar_done(p.ar_flags, q2, p.ar_max_tiles, out_tile), ar_epoch);
        }
      }
      if (p.ar_debug && ct == 0) p.ar_debug[(blockIdx.x * 16 + min(it - 1, 15)) * 4 + 3] = globaltimer_ns();
      if (p.ar_scatter) continue;
      // take one finished tile of a peer if its flag is already here
      const int pt = peer_tile(pull_u);
      if (ct == 0)
        *pull_ready = pt < out_tiles && flag_reached(ar_done(p.ar_flags, p.ar_rank, p.ar_max_tiles, pt), ar_epoch);
      if (!comm_sync()) break;
      if (*pull_ready) {
        copy_tile(pt);
        pull_u += gridDim.x;
      }
    }
    // final sweep: the tiles whose flags had not arrived yet
    if (!*abort_flag && !p.ar_scatter) {
      for (int pt = peer_tile(pull_u); pt < out_tiles; pull_u += gridDim.x, pt = peer_tile(pull_u)) {
        if (ct == 0 && !ar_wait_flag(ar_done(p.ar_flags, p.ar_rank, p.ar_max_tiles, pt), ar_epoch, p.ar_limit_ns, p.status))
          *abort_flag = 1;
        if (!comm_sync()) break;
        copy_tile(pt);
      }
    }
    }   // all-reduce / reduce-scatter forms
  }

  tc_fence_before();
  __syncthreads();
  if (AR && threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ar_epoch_word + 1, 1u) == gridDim.x - 1) {   // last CTA out: next call uses the next number
      ar_epoch_word[1] = 0u;
      __threadfence();
      if (p.ar_gather) {          // arrival counts back to zero for the next call
        uint32_t* arrived = ar_arrived(p.ar_flags, p.ar_rank, p.ar_max_tiles);
        for (int i = 0; i < m_tiles; ++i) arrived[i] = 0u;
        __threadfence();
      }
      // every read of this rank's staging slots is over: peers may push the next call's partials
      for (int q2 = 0; q2 < p.ar_world; ++q2)
        if (q2 != p.ar_rank) st_release_sys(ar_fin(p.ar_flags, q2, p.ar_max_tiles, p.ar_rank), ar_epoch);
      *reinterpret_cast<volatile uint32_t*>(ar_epoch_word) = ar_epoch;
    }
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
}

// out[r,c] = sum_s partial[s,r,c] (+ residual), summed in split order (deterministic)
template <bool OUT_F32>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ out, long long ldo,
                                     const __nv_bfloat16* __restrict__ residual, long long ldr, int M, int N,
                                     int split_k) {
  const long long n4 = static_cast<long long>(M) * (N / 4);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / (N / 4));
    const int col = static_cast<int>(i - static_cast<long long>(row) * (N / 4)) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < split_k; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partial + (static_cast<long long>(s) * M + row) * N + col);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (residual) {
      const __nv_bfloat16* rp = residual + static_cast<long long>(row) * ldr + col;
      acc.x += __bfloat162float(rp[0]); acc.y += __bfloat162float(rp[1]);
      acc.z += __bfloat162float(rp[2]); acc.w += __bfloat162float(rp[3]);
    }
    if (OUT_F32) {
      *reinterpret_cast<float4*>(static_cast<float*>(out) + static_cast<long long>(row) * ldo + col) = acc;
    } else {
      __nv_bfloat162 a = __floats2bfloat162_rn(acc.x, acc.y), b = __floats2bfloat162_rn(acc.z, acc.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&a);
      o.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(out) + static_cast<long long>(row) * ldo + col) = o;
    }
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess || !p)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 row-major [rows, cols] with row stride ld (elements); box = [box_rows, 64 cols].
bool make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

template <int BN, bool OUT_F32, bool HAS_RES>
const char* launch_bn(const GemmArgs& a, cudaStream_t stream) {
  using C = Cfg<BN>;
  CUtensorMap tmA, tmB, tmA2, tmB2;
  if (!make_map(&tmA, a.A, a.M, a.K, a.lda, BM)) return "cuTensorMapEncodeTiled failed for A";
  const long long b_rows = a.tile_expert ? static_cast<long long>(a.N) * (a.n_experts > 0 ? a.n_experts : 1) : a.N;
  if (a.tile_expert && (a.K2 > 0 || a.split_k > 1 || a.ar_world > 1)) return "grouped mode takes no side operand, k-split or all-reduce";
  if (!make_map(&tmB, a.B, b_rows, a.K, a.ldb, BN)) return "cuTensorMapEncodeTiled failed for B";
  if (a.K2 > 0) {
    if (!make_map(&tmA2, a.A2, a.M, a.K2, a.lda2, BM)) return "cuTensorMapEncodeTiled failed for A2";
    if (!make_map(&tmB2, a.B2, a.N, a.K2, a.ldb2, BN)) return "cuTensorMapEncodeTiled failed for B2";
  } else {
    tmA2 = tmA;
    tmB2 = tmB;
  }
  GemmParams p{};
  p.M = a.M; p.N = a.N; p.K = a.K; p.K2 = a.K2;
  p.out = a.out; p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual);
  p.ldo = a.ldo; p.ldr = a.ldr; p.status = a.status; p.group_m = 16;
  const int kb_total = (a.K + BK - 1) / BK + (a.K2 + BK - 1) / BK;
  int split = a.split_k > 1 ? a.split_k : 1;
  if (split > kb_total) split = kb_total;
  p.kb_per_split = (kb_total + split - 1) / split;
  p.split_k = (kb_total + p.kb_per_split - 1) / p.kb_per_split;   // no empty slices
  p.partial = a.partial;
  p.tile_expert = a.tile_expert;
  p.glu_act = a.glu_act;
  p.ss_in = a.ss_in; p.ss_parts = a.ss_parts; p.ss_ld = a.ss_ld; p.ss_inv_k = a.ss_inv_k; p.ss_eps = a.ss_eps;
  p.ss_out = a.ss_out;
  p.lp_mode = a.lp_mode; p.lp_targets = a.lp_targets; p.lp_inv_t = a.lp_inv_t; p.lp_cap = a.lp_cap; p.lp_col0 = a.lp_col0;
  p.lp_ws = reinterpret_cast<float2*>(a.lp_ws); p.lp_tl = a.lp_tl; p.lp_lse = a.lp_lse; p.lp_coef = a.lp_coef;
  if (p.lp_mode && (p.split_k > 1 || a.ar_world > 1 || a.tile_expert || a.glu_act || a.ss_in || a.ss_out || OUT_F32 || HAS_RES || BN != 256))
    return "log-prob epilogue: plain bf16 call with 256-wide tiles only";
  if (p.split_k > 1 && (!a.partial || (a.N % 4))) return "split-k needs a partial buffer and N % 4 == 0";
  p.ar_world = a.ar_world > 1 ? a.ar_world : 1;
  if (a.ar_gather) {
    if (p.ar_world < 2 || a.ar_world > kMaxRanks || a.ar_rank < 0 || a.ar_rank >= a.ar_world) return "all-gather GEMM: bad rank/world";
    if (a.M % (p.ar_world * BM) || a.M / BM > kMaxGatherMTiles || (a.K % 8) || a.lda != a.K || p.split_k > 1 || a.out_f32 ||
        a.A != a.ag_src.ptr[a.ar_rank])
      return "all-gather GEMM: M a multiple of world x 128 (at most 1024 row tiles), packed bf16 A in this rank's gather buffer, no split-k";
    p.ar_rank = a.ar_rank; p.ar_flags = a.ar_flags; p.ar_max_tiles = a.ar_max_tiles; p.ar_limit_ns = a.ar_limit_ns;
    p.ar_gather = 1; p.ag_src = a.ag_src;
  } else if (p.ar_world > 1) {
    if (a.out_f32 || p.split_k > 1 || (a.N % 8) || a.ldo != a.N) return "fused all-reduce needs bf16 output, no split-k, N % 8 == 0, packed output";
    const int out_tiles = ((a.M + BM - 1) / BM) * ((a.N + BN - 1) / BN);
    if (out_tiles > a.ar_max_tiles) return "fused all-reduce: flag buffer too small for this many tiles";
    const long long slots = static_cast<long long>((out_tiles + p.ar_world - 1) / p.ar_world) * p.ar_world;
    if (slots * BM * BN > a.ar_stage_elems || static_cast<long long>(a.M) * a.N > a.ar_out_elems)
      return "fused all-reduce: symmetric buffers too small for this output";
    if (a.residual && ((a.ldr % 8) || (reinterpret_cast<uintptr_t>(a.residual) & 15)))
      return "fused all-reduce: residual must be 16-byte aligned with ldr % 8 == 0";
    if (a.ar_world > kMaxRanks || a.ar_rank < 0 || a.ar_rank >= a.ar_world) return "fused all-reduce: bad rank/world";
    p.ar_rank = a.ar_rank; p.ar_stage = a.ar_stage; p.ar_outbuf = a.ar_outbuf;
    p.ar_flags = a.ar_flags; p.ar_max_tiles = a.ar_max_tiles; p.ar_limit_ns = a.ar_limit_ns;
    p.ar_debug = a.ar_debug;
    if ((a.ar_mc_stage != nullptr) != (a.ar_mc_outbuf != nullptr)) return "fused all-reduce: both multicast addresses or none";
    if (a.ar_mc_stage) {
      if (static_cast<long long>(out_tiles) * BM * BN > a.ar_stage_elems) return "fused all-reduce: staging buffer too small for one slot per tile";
      if ((reinterpret_cast<uintptr_t>(a.ar_mc_stage) & 15) || (reinterpret_cast<uintptr_t>(a.ar_mc_outbuf) & 15))
        return "fused all-reduce: multicast addresses must be 16-byte aligned";
    }
    p.ar_mc_stage = a.ar_mc_stage; p.ar_mc_outbuf = a.ar_mc_outbuf;
    if (a.ar_scatter) {
      if (a.M % (p.ar_world * BM) || a.residual || a.ar_mc_stage)
        return "fused reduce-scatter: M must be a multiple of world x 128; no residual, no multicast staging";
      p.ar_scatter = 1;
    }
  }
  constexpr bool kArOk = !OUT_F32 && (BN == 256 || BN == 128 || BN == 64);
  if (p.ar_world > 1 && !kArOk) return "fused all-reduce: unsupported tile width or output type";
  auto kern_plain = gemm_kernel<BN, OUT_F32, HAS_RES, false>;
  auto kern_ar = gemm_kernel<BN, OUT_F32, HAS_RES, kArOk>;      // same as plain when the mode is not available
  auto kern = p.ar_world > 1 ? kern_ar : kern_plain;
  if (!FERRL_ONCE_PER_DEVICE(
          cudaFuncSetAttribute(kern_plain, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) == cudaSuccess &&
          cudaFuncSetAttribute(kern_ar, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) == cudaSuccess))
    return "cudaFuncSetAttribute(max dynamic smem) failed";
  int m_tiles = (a.M + BM - 1) / BM, n_tiles = (a.N + BN - 1) / BN;
  int tiles = m_tiles * n_tiles * p.split_k;
  int grid = tiles < a.num_sms ? tiles : a.num_sms;
  if (grid < 1) return nullptr;
  p.pdl = (a.pdl && p.ar_world <= 1 && !p.tile_expert && p.split_k == 1) ? 1 : 0;
  if (p.pdl) {
    if (launch_pdl(kern, dim3(grid), dim3(NUM_THREADS), C::SMEM_BYTES, stream, tmA, tmB, tmA2, tmB2, p) != cudaSuccess)
      return "gemm launch (programmatic dependent) failed";
  } else {
    kern<<<grid, p.ar_world > 1 ? NUM_THREADS + 128 : NUM_THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, tmA2, tmB2, p);
  }
  count_launch();
  if (p.split_k > 1) {
    long long n4 = static_cast<long long>(a.M) * (a.N / 4);
    int rb = static_cast<int>((n4 + 255) / 256 < 148 * 8 ? (n4 + 255) / 256 : 148 * 8);
    if (OUT_F32)
      splitk_reduce_kernel<true><<<rb, 256, 0, stream>>>(a.partial, a.out, a.ldo, p.residual, a.ldr, a.M, a.N, p.split_k);
    else
      splitk_reduce_kernel<false><<<rb, 256, 0, stream>>>(a.partial, a.out, a.ldo, p.residual, a.ldr, a.M, a.N, p.split_k);
    count_launch();
  }
  return cudaGetLastError() == cudaSuccess ? nullptr : "gemm kernel launch failed";
}

// =============================================================================================
// Two-SM variant.  A cluster of two CTAs computes one 256 x BN tile with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and HALF of the B tile, so a
// k-block costs 32 KB of shared-memory fill per SM instead of 48 KB for the same tensor work.
// The one-SM kernel above is bound by that fill rate (about 64 B/clk/SM from L2) at ~70 % tensor
// activity on large problems; halving B's share lifts the bound above the tensor pipe's rate.
//
//   CTA 0 (leader)                          CTA 1
//   warp 0  TMA producer (own A, B half)    warp 0  TMA producer (own A, B half)
//   warp 1  MMA issuer for the pair         warp 1  (TMEM allocation only)
//   warps 2-5 epilogue of rows 0..127       warps 2-5 epilogue of rows 128..255
//
// Both producers' TMA loads (cta_group::2 form, no cluster multicast) complete their bytes on the
// LEADER's full barrier, which therefore expects two stages' worth per phase.  Stage release and
// accumulator-ready signals reach both CTAs through tcgen05.commit with a cluster multicast mask;
// the peer's epilogue warps release the accumulator with remote mbarrier arrives.  All waits are
// bounded as above.
template <int BN> struct Cfg2 {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN >= 256) ? 6 : 8;
  static constexpr int TMEM_COLS = (2 * BN <= 256) ? 256 : 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 512 /*barriers*/;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
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
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                  int code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        atomicCAS(status, kStatusOk, code);
        return false;
      }
    }
  }
  return true;
}
// TMA load whose completion is counted on a barrier that may live in the pair's other CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void umma2(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accum)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in every CTA of the mask when the MMAs retire
__device__ __forceinline__ void umma_commit2(uint64_t* bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(cta_mask)
               : "memory");
}
__host__ __device__ constexpr uint32_t make_idesc2(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(256 >> 4) << 24);
}

template <int BN, bool HAS_RES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
             const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2, GemmParams p,
             unsigned int* debug) {
  using C = Cfg2<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;                         // [STAGES] leader only: both CTAs' TMA bytes of the stage
  uint64_t* peer_full = bars + C::STAGES;        // [STAGES] unused (kept so the offsets match in both CTAs)
  uint64_t* empty = bars + 2 * C::STAGES;        // [STAGES] both CTAs: MMAs reading the stage retired
  uint64_t* acc_full = bars + 3 * C::STAGES;     // [2] both CTAs
  uint64_t* acc_empty = acc_full + 2;            // [2] leader only: 8 epilogue warps of the pair
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int m_tiles = (p.M + 2 * BM - 1) / (2 * BM);
  const int n_tiles = (p.N + BN - 1) / BN;
  const int total_tiles = m_tiles * n_tiles;
  const int kb1 = (p.K + BK - 1) / BK;
  const int kb2 = (p.K2 + BK - 1) / BK;
  const int kb_total = kb1 + kb2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&peer_full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers are initialised before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (debug && cluster == 0 && threadIdx.x == 0) debug[rank] = tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster; tile < total_tiles && ok; tile += num_clusters) {
        int mi, ni;
        tile_coords_mn(tile, m_tiles, n_tiles, p.group_m, mi, ni);
        const int a_row = mi * 2 * BM + static_cast<int>(rank) * BM;
        const int b_row = ni * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * C::STAGE_BYTES;
          uint8_t* sb = sa + C::A_BYTES;
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * C::STAGE_BYTES);
          const uint32_t bar = mapa_shared(smem_u32(&full[stage]), 0);
          if (kb < kb1) {
            tma_load_2d_pair(sa, &tmA, bar, kb * BK, a_row);
            tma_load_2d_pair(sb, &tmB, bar, kb * BK, b_row);
          } else {
            tma_load_2d_pair(sa, &tmA2, bar, (kb - kb1) * BK, a_row);
            tma_load_2d_pair(sb, &tmB2, bar, (kb - kb1) * BK, b_row);
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(10000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---------------------------------------------------------- MMA issuer (leader CTA)
      constexpr uint32_t idesc = make_idesc2(BN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int it = 0;
      bool ok = true;
      for (int tile = cluster; tile < total_tiles && ok; tile += num_clusters) {
        const int acc = (it++) & 1;
        if (!mbar_wait_cluster(&acc_empty[acc], acc_phase[acc] ^ 1, abort_flag, p.status, kStatusWaitTimeoutMma)) break;
        acc_phase[acc] ^= 1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait_cluster(&full[stage], phase, abort_flag, p.status, kStatusWaitTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
          const uint64_t da = make_smem_desc(sa);
          const uint64_t db = make_smem_desc(sb);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) umma2(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit2(&empty[stage], 3);     // frees the stage in both CTAs when these MMAs retire
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit2(&acc_full[acc], 3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (both CTAs)
    const int q = warp & 3;
    uint32_t acc_phase[2] = {0, 0};
    int it = 0;
    for (int tile = cluster; tile < total_tiles; tile += num_clusters) {
      int mi, ni;
      tile_coords_mn(tile, m_tiles, n_tiles, p.group_m, mi, ni);
      const int acc = (it++) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase[acc], abort_flag, p.status, kStatusWaitTimeoutEpilogue)) break;
      acc_phase[acc] ^= 1;
      tc_fence_after();
      const int row = mi * 2 * BM + static_cast<int>(rank) * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      LpRow lp;
      if (p.lp_mode) lp_begin(p, row, row_ok, lp);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c, r);
        tmem_ld_wait();
        const int col = ni * BN + c;
        if (row_ok && col < p.N) {
          const int ncols = min(min(32, BN - c), p.N - col);
          if (p.lp_mode) {
            lp_chunk(p, r, col, ncols, lp);
            if (p.lp_mode == 1) continue;
          }
          if (HAS_RES) {
            const __nv_bfloat16* rp = p.residual + static_cast<long long>(row) * p.ldr + col;
            if (ncols == 32 && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 x = reinterpret_cast<const uint4*>(rp)[v];
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  float2 f = __bfloat1622float2(h[e]);
                  r[v * 8 + 2 * e] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * e]) + f.x);
                  r[v * 8 + 2 * e + 1] = __float_as_uint(__uint_as_float(r[v * 8 + 2 * e + 1]) + f.y);
                }
              }
            } else {
              for (int e = 0; e < ncols; ++e)
                r[e] = __float_as_uint(__uint_as_float(r[e]) + __bfloat162float(rp[e]));
            }
          }
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldo + col;
          if (ncols == 32 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f8[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f8[e] = __uint_as_float(r[v * 8 + e]);
              reinterpret_cast<uint4*>(op)[v] = pack8(f8);
            }
          } else {
            for (int e = 0; e < ncols; ++e) op[e] = __float2bfloat16_rn(__uint_as_float(r[e]));
          }
        }
      }
      if (p.lp_mode) lp_end(p, row, row_ok, ni, lp);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(&acc_empty[acc]);
        else mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty[acc]), 0));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // the peer may still signal into, or the leader's MMAs read from, this CTA
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
}

template <int BN, bool HAS_RES>
const char* launch_2cta(const GemmArgs& a, cudaStream_t stream) {
  using C = Cfg2<BN>;
  CUtensorMap tmA, tmB, tmA2, tmB2;
  if (!make_map(&tmA, a.A, a.M, a.K, a.lda, BM)) return "cuTensorMapEncodeTiled failed for A";
  if (!make_map(&tmB, a.B, a.N, a.K, a.ldb, BN / 2)) return "cuTensorMapEncodeTiled failed for B";
  if (a.K2 > 0) {
    if (!make_map(&tmA2, a.A2, a.M, a.K2, a.lda2, BM)) return "cuTensorMapEncodeTiled failed for A2";
    if (!make_map(&tmB2, a.B2, a.N, a.K2, a.ldb2, BN / 2)) return "cuTensorMapEncodeTiled failed for B2";
  } else {
    tmA2 = tmA;
    tmB2 = tmB;
  }
  GemmParams p{};
  p.M = a.M; p.N = a.N; p.K = a.K; p.K2 = a.K2;
  p.out = a.out; p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual);
  p.ldo = a.ldo; p.ldr = a.ldr; p.status = a.status; p.group_m = 8;
  p.split_k = 1; p.ar_world = 1;
  p.lp_mode = a.lp_mode; p.lp_targets = a.lp_targets; p.lp_inv_t = a.lp_inv_t; p.lp_cap = a.lp_cap; p.lp_col0 = a.lp_col0;
  p.lp_ws = reinterpret_cast<float2*>(a.lp_ws); p.lp_tl = a.lp_tl; p.lp_lse = a.lp_lse; p.lp_coef = a.lp_coef;
  if (p.lp_mode && (HAS_RES || BN != 256)) return "log-prob epilogue: plain bf16 call with 256-wide tiles only";
  auto kern = gemm2_kernel<BN, HAS_RES>;
  if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) ==
                             cudaSuccess))
    return "cudaFuncSetAttribute(max dynamic smem) failed";
  const int m_tiles = (a.M + 2 * BM - 1) / (2 * BM), n_tiles = (a.N + BN - 1) / BN;
  const int tiles = m_tiles * n_tiles;
  int clusters = tiles < a.num_sms / 2 ? tiles : a.num_sms / 2;
  if (clusters < 1) return nullptr;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  unsigned int* dbg = a.debug;
  if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmA2, tmB2, p, dbg) != cudaSuccess) return "2-CTA gemm launch failed";
  count_launch();
  return nullptr;
}

// =============================================================================================
// Cluster split-K variant for decode-shaped problems (one or two M tiles, long K).
// A cluster of S CTAs shares one 128 x BN output tile: CTA r accumulates k-blocks
// [r*kb/S, (r+1)*kb/S) in TMEM, then the partial sums are exchanged through distributed shared
// memory as a reduce-scatter - CTA r receives every peer's partial of column slice r, adds the S
// partials in rank order (its own in its place, so the order does not depend on who adds) and
// writes that slice of the output.  One launch, no fp32 round trip through global memory, and the
// result is bit-identical from run to run.  Non-persistent: one k-slice of one tile per CTA.
template <int BN, int S> struct CfgK {
  static constexpr int STAGE_BYTES = (BM + BN) * BK * 2;
  static constexpr int SLICE = BN / S;                               // output columns owned by one CTA
  static constexpr int SLOT_BYTES = BM * SLICE * 4;                  // one peer's fp32 partial of my slice
  static constexpr int RED_BYTES = (S - 1) * SLOT_BYTES;
  static constexpr int STAGES_FIT = (220 * 1024 - RED_BYTES - 1024 - 256) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + RED_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void st_cluster_f4(uint32_t cluster_addr, float4 v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}

template <int BN, int S, bool OUT_F32, bool HAS_RES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_ksplit_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2, GemmParams p) {
  using C = CfgK<BN, S>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* red = reinterpret_cast<float*>(smem + C::STAGES * C::STAGE_BYTES);   // [S-1][BM][SLICE]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES + C::RED_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* acc_full = bars + 2 * C::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int tile = blockIdx.x / S;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int mi = tile / n_tiles, ni = tile % n_tiles;
  const int kb1 = (p.K + BK - 1) / BK;
  const int kb2 = (p.K2 + BK - 1) / BK;
  const int kb_total = kb1 + kb2;
  const int kb_per = (kb_total + S - 1) / S;
  const int kb_begin = min(kb_total, rank * kb_per), kb_end = min(kb_total, kb_begin + kb_per);
  if (threadIdx.x == 0) pdl_trigger();   // a dependent kernel may start its own prologue now

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int pre = 0;
      if (p.pdl) {
        pre = min(C::STAGES, kb_end - kb_begin);
        for (int i = 0; i < pre; ++i) {           // first pass over the ring: every stage is free
          const int kb = kb_begin + i;
          uint8_t* sb = smem + i * C::STAGE_BYTES + BM * BK * 2;
          mbar_expect_tx(&full[i], C::STAGE_BYTES);
          if (kb < kb1) tma_load_2d(sb, &tmB, &full[i], kb * BK, ni * BN);
          else tma_load_2d(sb, &tmB2, &full[i], (kb - kb1) * BK, ni * BN);
        }
        pdl_wait();
        for (int i = 0; i < pre; ++i) {
          const int kb = kb_begin + i;
          uint8_t* sa = smem + i * C::STAGE_BYTES;
          if (kb < kb1) tma_load_2d(sa, &tmA, &full[i], kb * BK, mi * BM);
          else tma_load_2d(sa, &tmA2, &full[i], (kb - kb1) * BK, mi * BM);
        }
        if (pre == C::STAGES) phase = 1; else stage = pre;
      }
      for (int kb = kb_begin + pre; kb < kb_end; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) {
          ok = false;
          break;
        }
        uint8_t* sa = smem + stage * C::STAGE_BYTES;
        uint8_t* sb = sa + BM * BK * 2;
        mbar_expect_tx(&full[stage], C::STAGE_BYTES);
        if (kb < kb1) {
          tma_load_2d(sa, &tmA, &full[stage], kb * BK, mi * BM);
          tma_load_2d(sb, &tmB, &full[stage], kb * BK, ni * BN);
        } else {
          tma_load_2d(sa, &tmA2, &full[stage], (kb - kb1) * BK, mi * BM);
          tma_load_2d(sb, &tmB2, &full[stage], (kb - kb1) * BK, ni * BN);
        }
        if (++stage == C::STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(10000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(&full[stage], phase, abort_flag, p.status, kStatusWaitTimeoutMma)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
        const uint32_t sb = sa + BM * BK * 2;
        const uint64_t da = make_smem_desc(sa);
        const uint64_t db = make_smem_desc(sb);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) umma(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
        umma_commit(&empty[stage]);
        if (++stage == C::STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(acc_full);
    }
  }

  // ---- exchange: every thread of the cluster passes the same two cluster barriers
  const bool epi = warp >= 2;
  const int q = warp & 3;
  const int row_in = q * 32 + lane;                 // accumulator row held by this thread
  const bool have = kb_end > kb_begin;              // a slice can be empty when kb_total < S
  bool acc_ok = true;
  float rstd = 1.f;
  if (epi && p.ss_in) {
    // gathered while the main loop runs (see row_rstd); the statistics come from the stream predecessor
    if (p.pdl) pdl_wait();
    if (mi * BM + row_in < p.M) rstd = row_rstd(p.ss_in, p.ss_parts, p.ss_ld, mi * BM + row_in, p.ss_inv_k, p.ss_eps);
  }
  if (epi) {
    if (have) acc_ok = mbar_wait(acc_full, 0, abort_flag, p.status, kStatusWaitTimeoutEpilogue);
    tc_fence_after();
    // push my partial of every other CTA's column slice into that CTA's receive slot [my rank]
    for (int dst = 0; dst < S; ++dst) {
      if (dst == rank) continue;
      const int slot = rank < dst ? rank : rank - 1;     // the receiver's slots skip its own rank
      const uint32_t base = mapa_shared(smem_u32(red + (static_cast<size_t>(slot) * BM + row_in) * C::SLICE), dst);
#pragma unroll 1
      for (int c = 0; c < C::SLICE; c += 16) {
        uint32_t r[16];
        if (have && acc_ok) {
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
              : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
              : "r"(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + dst * C::SLICE + c)
              : "memory");
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) r[e] = 0u;
        }
#pragma unroll
        for (int v = 0; v < 4; ++v)
          st_cluster_f4(base + (c + 4 * v) * 4, make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                            __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3])));
      }
    }
  }
  cluster_sync_all();                                 // all partials have landed in their owners' slots
  float ssq = 0.f;
  if (epi && acc_ok && !*abort_flag) {
    const int row = mi * BM + row_in;
    const int col0 = ni * BN + rank * C::SLICE;

#pragma unroll 1
    for (int c = 0; c < C::SLICE; c += 16) {
      uint32_t r[16];
      if (have) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + rank * C::SLICE + c)
            : "memory");
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) r[e] = 0u;
      }
      float acc[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) acc[e] = 0.f;
      for (int src = 0; src < S; ++src) {            // rank order, my own partial in its place
        if (src == rank) {
#pragma unroll
          for (int e = 0; e < 16; ++e) acc[e] += __uint_as_float(r[e]);
        } else {
          const int slot = src < rank ? src : src - 1;
          const float4* sp = reinterpret_cast<const float4*>(red + (static_cast<size_t>(slot) * BM + row_in) * C::SLICE + c);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const float4 x = sp[v];
            acc[4 * v] += x.x; acc[4 * v + 1] += x.y; acc[4 * v + 2] += x.z; acc[4 * v + 3] += x.w;
          }
        }
      }
      const int col = col0 + c;
      if (row < p.M && col < p.N) {
        const int ncols = min(16, p.N - col);
        if (p.ss_in) {
#pragma unroll
          for (int e = 0; e < 16; ++e) acc[e] *= rstd;
        }
        if (HAS_RES) {
          const __nv_bfloat16* rp = p.residual + static_cast<long long>(row) * p.ldr + col;
          for (int e = 0; e < ncols; ++e) acc[e] += __bfloat162float(rp[e]);
        }
        if (p.ss_out && !OUT_F32) {
          for (int e = 0; e < ncols; ++e) {
            const float hv = __bfloat162float(__float2bfloat16_rn(acc[e]));
            ssq += hv * hv;
          }
        }
        if (OUT_F32) {
          float* op = reinterpret_cast<float*>(p.out) + static_cast<long long>(row) * p.ldo + col;
          if (ncols == 16 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
#pragma unroll
            for (int v = 0; v < 4; ++v)
              reinterpret_cast<float4*>(op)[v] = make_float4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
          } else {
            for (int e = 0; e < ncols; ++e) op[e] = acc[e];
          }
        } else {
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldo + col;
          if (ncols == 16 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
            reinterpret_cast<uint4*>(op)[0] = pack8(acc);
            reinterpret_cast<uint4*>(op)[1] = pack8(acc + 8);
          } else {
            for (int e = 0; e < ncols; ++e) op[e] = __float2bfloat16_rn(acc[e]);
          }
        }
      }
    }
  }
  if (epi && acc_ok && !*abort_flag && p.ss_out && (mi * BM + row_in) < p.M)
    p.ss_out[(static_cast<long long>(ni) * S + rank) * p.ss_ld + mi * BM + row_in] = ssq;
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                 // nobody leaves while a peer may still read its slots' senders
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
}

template <int BN, int S, bool OUT_F32, bool HAS_RES>
const char* launch_ksplit(const GemmArgs& a, cudaStream_t stream) {
  using C = CfgK<BN, S>;
  static_assert(C::STAGES >= 3, "not enough shared memory left for the pipeline");
  static_assert(C::SLICE % 16 == 0, "column slice must be a multiple of 16");
  CUtensorMap tmA, tmB, tmA2, tmB2;
  if (!make_map(&tmA, a.A, a.M, a.K, a.lda, BM)) return "cuTensorMapEncodeTiled failed for A";
  if (!make_map(&tmB, a.B, a.N, a.K, a.ldb, BN)) return "cuTensorMapEncodeTiled failed for B";
  if (a.K2 > 0) {
    if (!make_map(&tmA2, a.A2, a.M, a.K2, a.lda2, BM)) return "cuTensorMapEncodeTiled failed for A2";
    if (!make_map(&tmB2, a.B2, a.N, a.K2, a.ldb2, BN)) return "cuTensorMapEncodeTiled failed for B2";
  } else {
    tmA2 = tmA;
    tmB2 = tmB;
  }
  GemmParams p{};
  p.M = a.M; p.N = a.N; p.K = a.K; p.K2 = a.K2;
  p.out = a.out; p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual);
  p.ldo = a.ldo; p.ldr = a.ldr; p.status = a.status; p.group_m = 1;
  p.split_k = 1; p.ar_world = 1;
  p.ss_in = a.ss_in; p.ss_parts = a.ss_parts; p.ss_ld = a.ss_ld; p.ss_inv_k = a.ss_inv_k; p.ss_eps = a.ss_eps;
  p.ss_out = a.ss_out;
  auto kern = gemm_ksplit_kernel<BN, S, OUT_F32, HAS_RES>;
  if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) ==
                             cudaSuccess))
    return "cudaFuncSetAttribute(max dynamic smem) failed";
  const int tiles = ((a.M + BM - 1) / BM) * ((a.N + BN - 1) / BN);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * S);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  p.pdl = a.pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmA2, tmB2, p) != cudaSuccess) return "cluster split-k gemm launch failed";
  count_launch();
  return nullptr;
}

template <int BN, int S>
const char* launch_ksplit_flags(const GemmArgs& a, cudaStream_t stream) {
  if (a.out_f32) return a.residual ? launch_ksplit<BN, S, true, true>(a, stream) : launch_ksplit<BN, S, true, false>(a, stream);
  return a.residual ? launch_ksplit<BN, S, false, true>(a, stream) : launch_ksplit<BN, S, false, false>(a, stream);
}

// =============================================================================================
// Stream-K variant for decode-shaped problems (one M tile): the n_tiles x k_blocks work units are
// dealt out as equal contiguous ranges, one per SM, so every SM streams the same number of weight
// bytes whatever N and K are; a range may start or end in the middle of a tile.
//
//   * whole tiles inside a range take the ordinary epilogue;
//   * a partial tile's fp32 accumulator is published row-major to a per-CTA workspace slot with a
//     release flag (the first and the last segment of a range can be partial: two slots per CTA);
//   * after its main loop, every contributor of a split tile waits for the others' flags and
//     finishes a band of ROWS of that tile: it adds the partials in k order (lower CTA index =
//     earlier k range, so the order is fixed), adds the residual and writes the output.
//
// Publishing never waits, so the waits cannot deadlock; they are bounded like all others.  One
// persistent launch pays the prologue once (the cluster split-k kernel pays it per wave) and the
// fix-up traffic stays in L2.  BN = 256 keeps the activation share of the fill at one third.
constexpr int SK_BN = 256;

struct StreamKParams {
  float* ws;                 // [grid][2][BM][SK_BN] fp32 partial tiles
  uint32_t* flags;           // [max_ctas][2] epochs, then [epoch word][done counter]
  uint32_t* epoch_ptr;       // device-resident launch counter: the kernel advances it itself, so a
  uint32_t* done_ptr;        //   captured CUDA graph can replay the launch (a host-side epoch would be baked in)
  long long units;           // n_tiles * kb_total
  unsigned long long* debug; // optional [grid][4] globaltimer stamps: start, last publish, flags seen, end
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <bool OUT_F32, bool HAS_RES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_streamk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2, GemmParams p,
                    StreamKParams sk) {
  constexpr int BN = SK_BN;
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* acc_full = bars + 2 * C::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint64_t* epi_bar = acc_empty + 3;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kb1 = (p.K + BK - 1) / BK;
  const int kb2 = (p.K2 + BK - 1) / BK;
  const int kb_total = kb1 + kb2;
  const int G = gridDim.x;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(sk.epoch_ptr) + 1;   // this launch's flag value
  if (sk.debug && threadIdx.x == 64) sk.debug[blockIdx.x * 4 + 0] = globaltimer_ns();
  auto range_lo = [&](int cta) -> long long { return static_cast<long long>(cta) * sk.units / G; };
  const long long u_lo = range_lo(blockIdx.x), u_hi = range_lo(blockIdx.x + 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    mbar_init(epi_bar, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(C::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long u = u_lo; u < u_hi && ok; ++u) {
        const int ni = static_cast<int>(u / kb_total), kb = static_cast<int>(u % kb_total);
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, p.status, kStatusWaitTimeoutProducer)) {
          ok = false;
          break;
        }
        uint8_t* sa = smem + stage * C::STAGE_BYTES;
        uint8_t* sb = sa + BM * BK * 2;
        mbar_expect_tx(&full[stage], C::STAGE_BYTES);
        if (kb < kb1) {
          tma_load_2d(sa, &tmA, &full[stage], kb * BK, 0);
          tma_load_2d(sb, &tmB, &full[stage], kb * BK, ni * BN);
        } else {
          tma_load_2d(sa, &tmA2, &full[stage], (kb - kb1) * BK, 0);
          tma_load_2d(sb, &tmB2, &full[stage], (kb - kb1) * BK, ni * BN);
        }
        if (++stage == C::STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        for (int i = 0; i < 64; ++i) __nanosleep(10000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int it = 0;
      bool ok = true;
      long long u = u_lo;
      while (u < u_hi && ok) {
        const long long tile_end = (u / kb_total + 1) * kb_total;
        const long long seg_end = tile_end < u_hi ? tile_end : u_hi;
        const int acc = (it++) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase[acc] ^ 1, abort_flag, p.status, kStatusWaitTimeoutMma)) break;
        acc_phase[acc] ^= 1;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (long long uu = u; uu < seg_end; ++uu) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, kStatusWaitTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + BM * BK * 2;
          const uint64_t da = make_smem_desc(sa);
          const uint64_t db = make_smem_desc(sb);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) umma(d_tmem, da + 2 * k, db + 2 * k, idesc, (uu > u || k > 0) ? 1u : 0u);
          umma_commit(&empty[stage]);
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&acc_full[acc]);
        u = seg_end;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int q = warp & 3;
    const int et = threadIdx.x - 64;
    uint32_t acc_phase[2] = {0, 0};
    int it = 0;
    uint32_t epi_phase = 0;
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(epi_bar);
      const bool ok = mbar_wait(epi_bar, epi_phase, abort_flag, p.status, kStatusWaitTimeoutEpilogue);
      epi_phase ^= 1;
      return ok && !*abort_flag;
    };
    int split_tile[2] = {-1, -1};          // tiles this CTA holds a partial of (slot 0: first segment, slot 1: last)
    bool live = true;
    long long u = u_lo;
    const int row = q * 32 + lane;         // single M tile: accumulator row == output row
    const bool row_ok = row < p.M;
    while (u < u_hi) {
      const int ni = static_cast<int>(u / kb_total);
      const long long tile_begin = static_cast<long long>(ni) * kb_total, tile_end = tile_begin + kb_total;
      const long long seg_end = tile_end < u_hi ? tile_end : u_hi;
      const bool whole = (u == tile_begin) && (seg_end == tile_end);
      const int acc = (it++) & 1;
      if (!mbar_wait(&acc_full[acc], acc_phase[acc], abort_flag, p.status, kStatusWaitTimeoutEpilogue)) {
        live = false;
        break;
      }
      acc_phase[acc] ^= 1;
      tc_fence_after();
      const int slot = (u == u_lo) ? 0 : 1;
      if (!whole) split_tile[slot] = ni;
      float* part = sk.ws + ((static_cast<long long>(blockIdx.x) * 2 + slot) * BM + row) * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c, r);
        tmem_ld_wait();
        if (!whole) {
#pragma unroll
          for (int v = 0; v < 8; ++v)
            reinterpret_cast<uint4*>(part + c)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
          continue;
        }
        const int col = ni * BN + c;
        if (row_ok && col < p.N) {
          const int ncols = min(32, p.N - col);
          if (HAS_RES) {
            const __nv_bfloat16* rp = p.residual + static_cast<long long>(row) * p.ldr + col;
            for (int e = 0; e < ncols; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) + __bfloat162float(rp[e]));
          }
          if (OUT_F32) {
            float* op = reinterpret_cast<float*>(p.out) + static_cast<long long>(row) * p.ldo + col;
            if (ncols == 32 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                reinterpret_cast<uint4*>(op)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
            } else {
              for (int e = 0; e < ncols; ++e) op[e] = __uint_as_float(r[e]);
            }
          } else {
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(row) * p.ldo + col;
            if (ncols == 32 && ((reinterpret_cast<uintptr_t>(op) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float f8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) f8[e] = __uint_as_float(r[v * 8 + e]);
                reinterpret_cast<uint4*>(op)[v] = pack8(f8);
              }
            } else {
              for (int e = 0; e < ncols; ++e) op[e] = __float2bfloat16_rn(__uint_as_float(r[e]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (!whole) {
        __threadfence();
        if (!epi_sync()) {
          live = false;
          break;
        }
        if (et == 0) {
          st_release_gpu(sk.flags + blockIdx.x * 2 + slot, epoch);
          if (sk.debug) sk.debug[blockIdx.x * 4 + 1] = globaltimer_ns();
        }
      }
      u = seg_end;
    }
    // ---- fix-up: finish a band of rows of every tile this CTA holds a partial of
    for (int sl = 0; sl < 2 && live; ++sl) {
      const int ni = split_tile[sl];
      if (ni < 0 || (sl == 1 && split_tile[0] == ni)) continue;
      const long long tb = static_cast<long long>(ni) * kb_total, te = tb + kb_total;
      // contributors: CTAs whose range intersects [tb, te)
      int c_first = static_cast<int>((tb * G) / sk.units);
      while (c_first > 0 && range_lo(c_first) > tb) --c_first;
      while (range_lo(c_first + 1) <= tb) ++c_first;
      int c_last = c_first;
      while (c_last + 1 < G && range_lo(c_last + 1) < te) ++c_last;
      const int n = c_last - c_first + 1, me = static_cast<int>(blockIdx.x) - c_first;
      if (et == 0) {
        const uint64_t t0 = globaltimer_ns();
        for (int c = c_first; c <= c_last; ++c) {
          const int cslot = (range_lo(c) >= tb) ? 0 : 1;     // the tile holds c's range start -> first segment
          uint32_t spins = 0;
          while (static_cast<int32_t>(ld_acquire_gpu(sk.flags + c * 2 + cslot) - epoch) < 0) {
            if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
              atomicCAS(p.status, kStatusOk, kStatusPeerWaitTimeout);
              *abort_flag = 1;
              break;
            }
          }
          if (*abort_flag) break;
        }
      }
      if (!epi_sync()) break;
      if (sk.debug && et == 0) sk.debug[blockIdx.x * 4 + 2] = globaltimer_ns();
      const int rows_per = (BM + n - 1) / n;
      const int r0 = me * rows_per, r1 = min(min(BM, p.M), r0 + rows_per);
      constexpr int CH = BN / 4;           // float4 chunks per row
      constexpr int MAXC = 16;             // contributors whose loads are kept in flight together
      // slot of every contributor, one bit each (bit set: the tile is that CTA's last segment)
      unsigned long long slot_bits = 0ull;
      for (int c = c_first; c <= c_last && c - c_first < 64; ++c)
        if (range_lo(c) < tb) slot_bits |= 1ull << (c - c_first);
      for (int i = et; i < (r1 - r0) * CH; i += 128) {
        const int rr = r0 + i / CH, ch = i % CH;
        const int col = ni * BN + ch * 4;
        if (col >= p.N) continue;
        float4 acc4 = make_float4(0.f, 0.f, 0.f, 0.f);
        const float4* base = reinterpret_cast<const float4*>(sk.ws + static_cast<long long>(rr) * BN) + ch;
        constexpr long long CTA_STRIDE4 = 2LL * BM * BN / 4, SLOT_STRIDE4 = static_cast<long long>(BM) * BN / 4;
        for (int c0 = 0; c0 < n; c0 += MAXC) {
          float4 v[MAXC];
#pragma unroll
          for (int k = 0; k < MAXC; ++k) {   // all loads first: the sum below must not serialise on L2 latency
            const int ci = c0 + k;
            if (ci < n)
              v[k] = __ldcg(base + (c_first + ci) * CTA_STRIDE4 + ((slot_bits >> (ci & 63)) & 1ull) * SLOT_STRIDE4);
          }
#pragma unroll
          for (int k = 0; k < MAXC; ++k) {   // contributor order == k order: fixed summation order
            if (c0 + k < n) {
              acc4.x += v[k].x; acc4.y += v[k].y; acc4.z += v[k].z; acc4.w += v[k].w;
            }
          }
        }
        float o4[4] = {acc4.x, acc4.y, acc4.z, acc4.w};
        const int ncols = min(4, p.N - col);
        if (HAS_RES) {
          const __nv_bfloat16* rp = p.residual + static_cast<long long>(rr) * p.ldr + col;
          for (int e = 0; e < ncols; ++e) o4[e] += __bfloat162float(rp[e]);
        }
        if (OUT_F32) {
          float* op = reinterpret_cast<float*>(p.out) + static_cast<long long>(rr) * p.ldo + col;
          for (int e = 0; e < ncols; ++e) op[e] = o4[e];
        } else {
          __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(rr) * p.ldo + col;
          if (ncols == 4 && ((reinterpret_cast<uintptr_t>(op) & 7) == 0)) {
            uint2 w;
            __nv_bfloat162* wh = reinterpret_cast<__nv_bfloat162*>(&w);
            wh[0] = __floats2bfloat162_rn(o4[0], o4[1]);
            wh[1] = __floats2bfloat162_rn(o4[2], o4[3]);
            *reinterpret_cast<uint2*>(op) = w;
          } else {
            for (int e = 0; e < ncols; ++e) op[e] = __float2bfloat16_rn(o4[e]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (sk.debug && threadIdx.x == 64) sk.debug[blockIdx.x * 4 + 3] = globaltimer_ns();
  if (threadIdx.x == 0) {
    // the last CTA to get here advances the launch counter; everyone has finished reading flags by then
    __threadfence();
    if (atomicAdd(sk.done_ptr, 1u) == static_cast<uint32_t>(G - 1)) {
      *sk.done_ptr = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(sk.epoch_ptr) = epoch;
    }
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
}

template <bool OUT_F32, bool HAS_RES>
const char* launch_streamk(const GemmArgs& a, cudaStream_t stream) {
  constexpr int BN = SK_BN;
  using C = Cfg<BN>;
  if (a.M > BM) return "stream-k gemm: one M tile only";
  if (!a.sk_ws || !a.sk_flags) return "stream-k gemm: workspace missing";
  CUtensorMap tmA, tmB, tmA2, tmB2;
  if (!make_map(&tmA, a.A, a.M, a.K, a.lda, BM)) return "cuTensorMapEncodeTiled failed for A";
  if (!make_map(&tmB, a.B, a.N, a.K, a.ldb, BN)) return "cuTensorMapEncodeTiled failed for B";
  if (a.K2 > 0) {
    if (!make_map(&tmA2, a.A2, a.M, a.K2, a.lda2, BM)) return "cuTensorMapEncodeTiled failed for A2";
    if (!make_map(&tmB2, a.B2, a.N, a.K2, a.ldb2, BN)) return "cuTensorMapEncodeTiled failed for B2";
  } else {
    tmA2 = tmA;
    tmB2 = tmB;
  }
  GemmParams p{};
  p.M = a.M; p.N = a.N; p.K = a.K; p.K2 = a.K2;
  p.out = a.out; p.residual = reinterpret_cast<const __nv_bfloat16*>(a.residual);
  p.ldo = a.ldo; p.ldr = a.ldr; p.status = a.status; p.group_m = 1; p.split_k = 1; p.ar_world = 1;
  const int kb_total = (a.K + BK - 1) / BK + (a.K2 + BK - 1) / BK;
  const int n_tiles = (a.N + BN - 1) / BN;
  StreamKParams sk{};
  sk.ws = a.sk_ws; sk.flags = a.sk_flags;
  sk.epoch_ptr = a.sk_flags + 2 * a.sk_max_ctas;
  sk.done_ptr = a.sk_flags + 2 * a.sk_max_ctas + 1;
  sk.units = static_cast<long long>(n_tiles) * kb_total;
  sk.debug = a.sk_debug;
  int grid = a.num_sms < a.sk_max_ctas ? a.num_sms : a.sk_max_ctas;
  if (sk.units < grid) grid = static_cast<int>(sk.units);
  if (grid < 1) return nullptr;
  auto kern = gemm_streamk_kernel<OUT_F32, HAS_RES>;
  if (!FERRL_ONCE_PER_DEVICE(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) ==
                             cudaSuccess))
    return "cudaFuncSetAttribute(max dynamic smem) failed";
  kern<<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, tmA2, tmB2, p, sk);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? nullptr : "stream-k gemm launch failed";
}

template <int BN>
const char* launch_flags(const GemmArgs& a, cudaStream_t stream) {
  if (a.out_f32) return a.residual ? launch_bn<BN, true, true>(a, stream) : launch_bn<BN, true, false>(a, stream);
  return a.residual ? launch_bn<BN, false, true>(a, stream) : launch_bn<BN, false, false>(a, stream);
}

}  // namespace

int gemm_pick_bn(int M, int N, int num_sms) {
  // Large problems take the widest tile; when that leaves SMs idle shrink BN so that the
  // tile count approaches the SM count (decode-shaped GEMMs are bandwidth bound).
  int m_tiles = (M + BM - 1) / BM;
  const int cands[4] = {256, 128, 64, 32};
  for (int i = 0; i < 4; ++i) {
    int bn = cands[i];
    if (bn > 32 && N < bn) continue;
    long long tiles = static_cast<long long>(m_tiles) * ((N + bn - 1) / bn);
    if (tiles >= num_sms || bn == 32) return bn;
  }
  return 32;
}

// Decode-shaped problems (one or two M tiles) are bound by how many bytes each SM has to pull
// through its TMA path (about 64 GB/s per SM when the weights stream from HBM), not by HBM itself:
// pick the tile width and the k-split that minimise the bytes of the busiest SM (A slice + B slice
// per tile, times the number of waves).  Splits inside a cluster reduce through shared memory;
// the global-memory split (fp32 partials + reduce kernel) is the fallback.
void gemm_plan(int M, int N, int K, int K2, int num_sms, int* bn_out, int* split_out, int* cluster_out, double* est_out) {
  const int m_tiles = (M + BM - 1) / BM;
  *bn_out = gemm_pick_bn(M, N, num_sms);
  *split_out = 1;
  *cluster_out = 1;
  if (est_out) *est_out = 1e30;
  if (m_tiles > 2 || (N % 4)) return;
  const int kb_total = (K + BK - 1) / BK + (K2 + BK - 1) / BK;
  double best = 1e30;
  const int cands[4] = {256, 176, 128, 64};   // 176 exists to fit N = 24576 onto 140 of 148 SMs in one wave
  for (int ci = 0; ci < 4; ++ci) {
    const int bn = cands[ci];
    if (N < bn) continue;
    const int n_tiles = (N + bn - 1) / bn;
    for (int split = 1; split <= 16 && split <= kb_total; ++split) {
      if (bn == 176 && split > 1) break;
      const int per = (kb_total + split - 1) / split;
      const int eff = (kb_total + per - 1) / per;
      const long long tiles = static_cast<long long>(m_tiles) * n_tiles * eff;
      const long long waves = (tiles + num_sms - 1) / num_sms;
      double bytes = static_cast<double>(waves) * (BM + bn) * per * BK * 2.0;
      double t = bytes / 64e9 + 7e-6;                                 // one prologue/drain for the persistent kernel
      if (eff > 1) t += 8e-6 + static_cast<double>(M) * N * 4.0 * (eff + 1) / 5e12;   // partial write + reduce launch
      if (t < best) { best = t; *bn_out = bn; *split_out = eff; *cluster_out = 1; }
    }
    // cluster split: one CTA per k-slice, non-persistent
    const int cl[3] = {2, 4, 8};
    for (int k = 0; k < 3; ++k) {
      const int S = cl[k];
      const bool supported = (bn == 64 && S <= 4) || (bn == 128) || (bn == 256 && S == 2);
      if (!supported || S > kb_total || (N % 16)) continue;
      const int per = (kb_total + S - 1) / S;
      const long long ctas = static_cast<long long>(m_tiles) * n_tiles * S;
      const long long waves = (ctas + num_sms - 1) / num_sms;
      // measured: a cluster CTA pays ~9 us of prologue, exchange and drain per wave (one-tile CTAs
      // cannot hide it behind the next tile the way the persistent kernel does)
      double t = static_cast<double>(waves) * ((BM + bn) * static_cast<double>(per) * BK * 2.0 / 64e9 + 9e-6) + 1e-6;
      if (t < best) { best = t; *bn_out = bn; *split_out = 1; *cluster_out = S; }
    }
  }
  if (est_out) *est_out = best;
}

const char* gemm_bf16(const GemmArgs& a, cudaStream_t stream) {
  if (a.M <= 0 || a.N <= 0) return nullptr;
  if (a.K <= 0) return "K must be > 0";
  if ((a.K % 8) || (a.lda % 8) || (a.ldb % 8)) return "K and operand row strides must be multiples of 8 elements";
  if (a.K2 > 0 && ((a.K2 % 8) || (a.lda2 % 8) || (a.ldb2 % 8)))
    return "K2 and side-operand row strides must be multiples of 8 elements";
  if ((reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15) ||
      (a.K2 > 0 && ((reinterpret_cast<uintptr_t>(a.A2) & 15) || (reinterpret_cast<uintptr_t>(a.B2) & 15))))
    return "operand base addresses must be 16-byte aligned";
  if (a.ss_in || a.ss_out) {
    if (a.stream_k || a.two_cta || a.split_k > 1 || a.out_f32 || a.ar_world > 1 || a.tile_expert)
      return "gemm with folded RMSNorm: one-SM or cluster split-k kernel, bf16 output, no global split or grouping";
  }
  if (a.glu_act) {
    if (a.stream_k || a.cluster_k > 1 || a.two_cta || a.split_k > 1 || a.out_f32 || a.residual || a.ar_world > 1 || a.tile_expert ||
        (a.N % 16) || (a.ldo % 8))
      return "gemm with GLU epilogue: one-SM kernel, bf16 output, no split, residual or grouping; N a multiple of 16";
  }
  if (a.lp_mode) {
    if (a.stream_k || a.cluster_k > 1 || a.out_f32 || a.residual || a.K2 > 0 || !a.lp_targets ||
        (a.lp_mode == 1 && (!a.lp_ws || !a.lp_tl)) || (a.lp_mode == 2 && (!a.lp_lse || !a.lp_coef || !a.out)))
      return "log-prob epilogue: plain call (no side operand, residual or fp32 output) with its buffers set";
  }
  if (a.stream_k) {
    if (a.split_k > 1 || a.tile_expert || a.ar_world > 1) return "stream-k gemm: no global k-split, grouping or all-reduce";
    if (a.out_f32) return a.residual ? launch_streamk<true, true>(a, stream) : launch_streamk<true, false>(a, stream);
    return a.residual ? launch_streamk<false, true>(a, stream) : launch_streamk<false, false>(a, stream);
  }
  if (a.cluster_k > 1) {
    if (a.split_k > 1 || a.tile_expert || a.ar_world > 1) return "cluster split-k gemm: no global k-split, grouping or all-reduce";
    const int key = a.force_bn * 10 + a.cluster_k;
    switch (key) {
      case 642: return launch_ksplit_flags<64, 2>(a, stream);
      case 644: return launch_ksplit_flags<64, 4>(a, stream);
      case 1282: return launch_ksplit_flags<128, 2>(a, stream);
      case 1284: return launch_ksplit_flags<128, 4>(a, stream);
      case 1288: return launch_ksplit_flags<128, 8>(a, stream);
      case 2562: return launch_ksplit_flags<256, 2>(a, stream);
      default: return "cluster split-k gemm: unsupported (BN, cluster) pair";
    }
  }
  if (a.two_cta) {
    if (a.out_f32 || a.split_k > 1 || a.tile_expert || a.ar_world > 1) return "2-CTA gemm: bf16 output, no k-split, grouping or all-reduce";
    if (a.two_cta == 128) return a.residual ? launch_2cta<128, true>(a, stream) : launch_2cta<128, false>(a, stream);
    return a.residual ? launch_2cta<256, true>(a, stream) : launch_2cta<256, false>(a, stream);
  }
  int bn = a.force_bn > 0 ? a.force_bn : gemm_pick_bn(a.M, a.N, a.num_sms);
  switch (bn) {
    case 256: return launch_flags<256>(a, stream);
    case 176: return launch_flags<176>(a, stream);
    case 128: return launch_flags<128>(a, stream);
    case 64: return launch_flags<64>(a, stream);
    case 32: return launch_flags<32>(a, stream);
    default: return "unsupported BN";
  }
}

}  // namespace ferrl
