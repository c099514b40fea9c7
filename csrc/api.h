// Host-callable launchers of the sm_100a kernels. Every launcher takes raw device pointers
// plus a stream, returns nullptr on success or a static error string, and never allocates.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include <cuda_bf16.h>

#include "symm/symm.cuh"

namespace ferrl {

enum { kBF16 = 0, kF32 = 1 };
enum { kActSilu = 0, kActGeluTanh = 1 };

// ---- tcgen05 GEMM: out[M,N] = A[M,K] B[N,K]^T (+ A2[M,K2] B2[N,K2]^T) (+ residual) ----
struct GemmArgs {
  const void* A; const void* B; const void* A2; const void* B2;  // bf16, K-major
  long long lda, ldb, lda2, ldb2;                                 // row strides in elements
  int M, N, K, K2;
  void* out; long long ldo; bool out_f32;
  const void* residual; long long ldr;                            // optional bf16 [M, ldr]
  int* status;                                                    // device status word (kStatus*)
  int num_sms;
  int force_bn;                                                   // 0 = heuristic
  int split_k;                                                    // <= 1: none
  float* partial;                                                 // [split_k, M, N] fp32 scratch when split_k > 1
  // two-SM kernel (cluster of 2 CTAs, 256 x two_cta tiles): two_cta = 0 (off), 128 or 256
  int two_cta; unsigned int* debug;
  // cluster split-k kernel (decode shapes): cluster_k CTAs share one 128 x force_bn tile; 0/1 = off
  int cluster_k;
  // stream-k kernel (decode shapes, M <= 128): equal unit ranges per SM, partial tiles fixed up through `sk_ws`
  int stream_k; float* sk_ws; unsigned int* sk_flags; int sk_max_ctas; unsigned long long* sk_debug;
  // grouped mode: B is [n_experts * N, K]; tile_expert[m tile] = expert (or -1: skip the tile)
  const int* tile_expert; int n_experts;
  // fused GEMM -> all-reduce over the symmetric heap (ar_world > 1): see tcgen05_gemm.cu
  int ar_world, ar_rank; int ar_max_tiles; unsigned long long ar_limit_ns;
  long long ar_stage_elems, ar_out_elems;                         // capacity of the symmetric staging / output buffers (bf16 elements)
  PeerTable ar_stage, ar_outbuf, ar_flags;
  unsigned long long* ar_debug;
  // in-switch variant: multicast addresses of ar_stage / ar_outbuf (both or none), see GemmParams in tcgen05_gemm.cu
  void* ar_mc_stage; void* ar_mc_outbuf;
  // reduce-scatter form: rank r keeps rows [r M/world, (r+1) M/world) of the sum in `out` [M/world, N] and nothing is sent back
  // (M a multiple of world x 128, no residual, peer-load staging only)
  int ar_scatter;
  // all-gather -> GEMM (ar_gather != 0, with ar_world / ar_rank / ar_flags / ar_max_tiles / ar_limit_ns): A is this rank's
  // gather buffer ag_src.ptr[ar_rank], [M, K] packed, of which only its own M / world rows are filled; the kernel's
  // communication warps pull the other rows from the peers' buffers while the tensor cores work on the rows in place
  int ar_gather;
  PeerTable ag_src;
  // launch as a programmatic dependent of the stream predecessor: weights are prefetched before the
  // dependency wait (only where B is never written by an earlier kernel of the same stream)
  int pdl;
  // GLU epilogue: B rows interleaved in groups of 16 (8 gate, 8 up); out is [M, N/2]; 1 SiLU, 2 tanh-GELU
  int glu_act;
  // RMSNorm folded around the projection (one-SM and cluster split-k kernels, bf16 output):
  // ss_in [ss_parts, ss_ld] fp32 partial row sums of squares of A's rows (rows are scaled by
  // rsqrt(sum * ss_inv_k + ss_eps) in the epilogue); ss_out [parts, ss_ld] receives the partial row sums
  // of squares of the stored output, parts = gemm_ss_parts()
  const float* ss_in; int ss_parts; long long ss_ld; float ss_inv_k, ss_eps;
  float* ss_out;
  // language-model head without a logits tensor (tile width 256; two_cta 256 or the one-SM kernel):
  // every accumulator value x becomes the scored logit z = softcap(x) * lp_inv_t.
  // lp_mode 1: out is not written; lp_ws [ceil(N/256), M] float2 receives per row and column tile the running
  //            (max, sum exp(z - max)), lp_tl [M] the z of the target column (lp_targets int64, vocabulary index);
  // lp_mode 2: out (bf16) receives lp_coef[row] * (exp(z - lp_lse[row]) - [col == target]) * dz/dx.
  // B may be a slice of the vocabulary starting at row lp_col0.
  int lp_mode; const long long* lp_targets; float lp_inv_t, lp_cap; long long lp_col0;
  float* lp_ws; float* lp_tl; const float* lp_lse; const float* lp_coef;
};
// number of partial rows ss_out needs for a call that would run with tile width bn and cluster size (1: none)
inline int gemm_ss_parts(int N, int bn, int cluster) { return ((N + bn - 1) / bn) * (cluster > 1 ? cluster : 1); }
void gemm_plan(int M, int N, int K, int K2, int num_sms, int* bn_out, int* split_out, int* cluster_out,
               double* est_out = nullptr);
const char* gemm_bf16(const GemmArgs& a, cudaStream_t stream);
int gemm_pick_bn(int M, int N, int num_sms);

// ---- decode projection with resident activations (csrc/gemm/decode_gemm.cu): M <= 128, bf16 out ----
struct DecodeGemmArgs {
  const void* A; const void* B;            // bf16, K-major: A [M, K] activations, B [N, K] weights
  long long lda, ldb;
  int M, N, K;
  void* out; long long ldo;                // bf16 [M, N], or [M, N/2] with the GLU epilogue
  const void* residual; long long ldr;     // optional bf16 [M, N]
  int glu_act;                             // 0 none, 1 SiLU, 2 tanh-GELU (B rows interleaved in groups of 16: 8 gate, 8 up)
  float* partial;                          // fp32 [groups, M, N] scratch, needed when decode_gemm_groups(K) > 1
  int* status;                             // device status word (kStatus*)
  int pdl;                                 // programmatic dependent launch: B is never written by an earlier kernel
  int max_clusters;                        // 0 = as many as the device holds
  unsigned long long* debug;               // optional [64]: time stamps of one epilogue warp (development aid)
};
bool decode_gemm_supported(int M, int N, int K, bool glu);
int decode_gemm_groups(int K);
const char* decode_gemm(const DecodeGemmArgs& a, cudaStream_t stream);

// ---- norms / rope ----
const char* rmsnorm(int dtype, const void* x, const void* res, const void* w, const void* gate, void* y, void* h_out,
                    long long rows, int H, float eps, bool zero_centered, cudaStream_t s);
const char* rmsnorm_bwd(int dtype, const void* x, const void* w, const void* dy, void* dx, long long rows, int H,
                        float eps, bool zero_centered, cudaStream_t s);
// gated form y = rmsnorm(x) * w * silu(gate): gradients of x and gate for a frozen weight
const char* rmsnorm_gated_bwd(int dtype, const void* x, const void* gate, const void* w, const void* dy, void* dx,
                              void* dg, long long rows, int H, float eps, cudaStream_t s);
struct QkNormRopeArgs {
  int dtype; bool backward;
  const void* q_in; long long ld_q;                     // [n_tok, Hq*D] rows with token stride ld_q (may be a view
  const void* k_in; long long ld_k;                     //  into the fused qkv projection output)
  const void* qw; const void* kw;                       // per-head norm weights or nullptr
  const float* cos_t; const float* sin_t;               // [max_pos, half]
  const long long* pos64; const int* pos32; int pos_div; // position of token t is pos[t / pos_div]
  void* q_out; void* k_out;     // forward: contiguous [n_tok,Hq,D] / [n_tok,Hkv,D]; backward: d(q_in) / d(k_in)
  long long ld_dq, ld_dk;       // backward: token strides of the two gradient destinations
  const void* dq; const void* dk;                       // backward inputs (contiguous)
  long long n_tok; int Hq, Hkv, D, half; float eps; bool zero_centered;
  // decode (forward, one token per row, vector kernel only): when kc is set the rotated K row and
  // the V row of token t go straight to cache row kv_len[t] of sequence t (k_out is not written):
  // dense caches [B, smax, Hkv, D], or pools [n_pages, page, Hkv, D] behind table[t, kv_len / page]
  void* kc; void* vc; const void* v_in; long long ld_v;
  const int* kv_len; const int* table; int bt_stride, page, smax;
};
const char* qk_norm_rope(const QkNormRopeArgs& a, cudaStream_t s);
const char* row_sumsq(const void* x, long long ld, float* ss, int rows, int H, cudaStream_t s);   // bf16 rows
const char* kv_append_paged(const void* k, const void* v, long long ldv, void* kc, void* vc, const int* kv_len,
                            const int* table, int bt_stride, int page, int batch, int HD, cudaStream_t s);
const char* kv_append(int dtype, const void* k, const void* v, long long ldv, void* kc, void* vc, const int* kv_len,
                      int batch, int smax, int HD, cudaStream_t s);

// ---- misc ----
const char* glu(int dtype, bool backward, const void* gu, const void* dout, void* out, long long rows, int F, int act,
                cudaStream_t s);
const char* embedding(int dtype, const long long* ids, const void* table, void* out, long long n_tok, int H,
                      long long vocab, float scale, cudaStream_t s);
const char* lora_merge(int dtype, const void* w, const float* a, const float* b, void* out, int O, int I, int R,
                       cudaStream_t s);
struct AdamTensor { float* p; const float* g; float* m; float* v; long long n; };
const char* adamw_multi(const AdamTensor* tab_dev, const int* blk_tensor_dev, const long long* blk_off_dev,
                        int n_blocks, int chunk, double* sumsq_dev, bool compute_norm, float lr, float b1, float b2,
                        float eps, float wd, float bc1_inv, float bc2_inv, float max_norm, float pre_scale,
                        float* norm_out_dev, cudaStream_t s);
const char* grpo_loss_rows(const float* logp, const float* logp_old, const float* logp_ref, const float* adv,
                           const float* mask, const float* tis, float* row_sum, float* row_cnt, float* dlogp, int G,
                           int L, float eps_lo, float eps_hi, float beta, int mode, cudaStream_t s);
const char* grpo_scale_rows(float* dlogp, const float* row_scale, int G, int L, cudaStream_t s);

// ---- data-parallel fused step and symmetric-heap collectives ----
struct DpStepParams {
  PeerTable grads, reduced, flags, scalars;  // per-rank copies of the symmetric buffers
  int rank, world, barrier_world, own_lo, own_hi;
  long long n;                               // flat length, padded to a multiple of 4*world
  unsigned epoch; float pre_scale; float uncovered_local;
  const AdamTensor* tab; const int* blk_tensor; const long long* blk_off; const long long* blk_flat;
  int n_blocks, chunk;
  float lr, b1, b2, eps, wd, bc1_inv, bc2_inv, max_norm;
  double* block_partials;                    // local scratch, 2 doubles per block
  float* out;                                // [norm, uncovered_total, stepped]
  int* status; int* abort_word; unsigned long long limit_ns;
};
const char* dp_step(const DpStepParams& p, int num_sms, cudaStream_t s);
int dp_step_grid(int num_sms);
const char* symm_all_reduce(int dtype, const PeerTable& src, const PeerTable& flags, void* out, long long n, int rank,
                            int world, unsigned epoch, unsigned long long limit_ns, int* status, int* abort_word,
                            int num_sms, cudaStream_t s);
// The halves of that all-reduce for sequence-sharded tensor parallelism: which = 0 reduce-scatter (src: every rank's
// full partial [world * n_shard], out: this rank's summed slice [n_shard]); 1 all-gather (src: every rank's shard,
// out: all rows [world * n_shard]).
const char* symm_row_collective(int which, int dtype, const PeerTable& src, const PeerTable& flags, void* out, long long n_shard,
                                int rank, int world, unsigned epoch, unsigned long long limit_ns, int* status, int* abort_word,
                                int num_sms, cudaStream_t s);
// NVLS form (csrc/symm/nvls_all_reduce.cu): `mc` is the multicast address of the symmetric buffer whose local
// copy is `local`; in place in the buffer, then copied to `out`.  nbytes a multiple of 16 * world.
const char* nvls_all_reduce(int dtype, void* mc, const void* local, const PeerTable& flags, void* out, long long nbytes, int rank,
                            int world, unsigned epoch, unsigned long long limit_ns, int* status, int* abort_word, int num_sms,
                            cudaStream_t s);

// ---- decode attention ----
struct DecodeAttnArgs {
  const void* q; const void* k; const void* v;  // q [B,Hq,D]; caches [B,Smax,Hkv,D] (or paged)
  const int* kv_len; const int* block_table; int bt_stride, page;
  void* out; float* workspace;
  int B, Hq, Hkv, D; long long seq_stride, tok_stride; float scale; int window, n_splits;
  int no_pipe;   // 0: tensor-core pipelined kernel; 2: scalar pipelined kernel; 1: register-resident kernel
  // shared-prefix mode (paged cache, rows in groups of `group` that share their first prefix_len[b / group]
  // keys): those keys are streamed once per group; workspace: B * Hq * prefix_splits * (D + 2) floats
  const int* prefix_len; int group; int prefix_splits;
};
const char* decode_attn(const DecodeAttnArgs& a, cudaStream_t s);
size_t decode_attn_workspace_bytes(int B, int Hq, int D, int n_splits);
int decode_attn_pick_splits(int B, int Hkv, int max_len, int num_sms);

// ---- flash attention (prefill / training) ----
struct FlashArgs {
  const void* q; const void* k; const void* v; void* o; float* lse;   // bf16; lse [B,Hq,Sq]
  long long q_bs, q_ts, k_bs, k_ts, v_bs, v_ts, o_bs, o_ts;            // batch / token strides (elements)
  int B, Sq, Sk, Hq, Hkv, D; float scale; int causal, window, q_offset;
  // backward only
  const void* d_o; void* dq; void* dk; void* dv; float* delta;
  long long do_bs, do_ts, dq_bs, dq_ts, dk_bs, dk_ts, dv_bs, dv_ts;
  unsigned long long* debug;   // optional time stamps (tcgen05 backward), else null
};
const char* flash_fwd(const FlashArgs& a, cudaStream_t s);
const char* flash_bwd(const FlashArgs& a, cudaStream_t s);
// tcgen05 forward for causal self-attention with head_dim 128 (csrc/kernels/flash_tc.cu)
bool flash_fwd_tc_supported(const FlashArgs& a);
size_t flash_fwd_tc_workspace_elems(const FlashArgs& a);
const char* flash_fwd_tc(const FlashArgs& a, void* vt_ws, int* status, cudaStream_t stream, int form = 1);
// tcgen05 backward for the same domain (csrc/kernels/flash_bwd_tc.cu)
bool flash_bwd_tc_supported(const FlashArgs& a);
size_t flash_bwd_tc_scratch_floats(const FlashArgs& a);   // size of a.delta for flash_bwd_tc
const char* flash_bwd_tc(const FlashArgs& a, int* status, cudaStream_t stream);

// ---- vocabulary rows ----
// finish of the head GEMM's log-prob epilogue (GemmArgs::lp_mode 1): ws [n_tiles, M] float2, tl [M]
// the same combine for one vocabulary shard: stats [M, 3] = (max, sum exp(z - max), target logit or 0)
const char* logprob_shard_stats(const float* ws, const float* tl, int n_tiles, int M, float* stats, cudaStream_t s);
const char* logprob_finalize(const float* ws, const float* tl, int n_tiles, int M, float* lp, float* lse, cudaStream_t s);
const char* logprob_rows(int dtype, const void* logits, long long ld, const long long* targets, float* lp, float* lse,
                         long long rows, int V, float temperature, float softcap, cudaStream_t s);
const char* logprob_rows_bwd(int dtype, void* logits, long long ld, const long long* targets, const float* lse,
                             const float* dlp, long long rows, int V, float temperature, float softcap, cudaStream_t s);
const char* sample_rows(int dtype, const void* logits, long long ld, const long long* global_rows,
                        unsigned long long seed, const int* draw_dev, int draw_host, long long* tok_out, float* lp_out,
                        int rows, int V, float temperature, float top_p, cudaStream_t s);

// ---- mixture of experts (csrc/moe/moe.cu); all return nullptr on success
const char* moe_route(const float* logits, long long ld, int T, int E, int k, bool renorm, float* probs, float* scores,
                      int* idx, int* counts, cudaStream_t stream);
const char* moe_plan(const int* idx, const int* counts, int n_pairs, int k, int E, int max_rows, int* row_of,
                     int* token_of, int* tile_expert, int* seg_start, cudaStream_t stream);
const char* moe_gather(const void* x, long long ldx, const int* token_of, const float* pair_w, const int* row_of,
                       int n_pairs, float* row_scale, int rows, int H, void* xs, cudaStream_t stream);
const char* moe_combine(const void* ys, const int* row_of, const float* w, int T, int k, int H, void* out,
                        cudaStream_t stream);
const char* moe_pair_dot(const void* dy, const void* ys, const int* row_of, int n_pairs, int k, int H, float* dw,
                         cudaStream_t stream);

// ---- GatedDeltaNet (csrc/kernels/gdn.cu)
const char* gdn_conv_fwd(const void* x, long long ldx, const void* w, const void* left, int B, int L, int C, int K,
                         bool act, void* y, cudaStream_t stream);
const char* gdn_conv_bwd(const void* x, long long ldx, const void* w, const void* left, const void* dy, int B, int L,
                         int C, int K, bool act, void* dx, cudaStream_t stream);
const char* gdn_conv_step(const void* x, long long ldx, const void* w, void* state, int B, int C, int K, bool act,
                          void* y, cudaStream_t stream);
const char* gdn_chunk_fwd(const void* q, const void* k, const void* v, long long q_bs, long long q_ts, long long k_bs,
                          long long k_ts, long long v_bs, long long v_ts, const float* g, const float* beta,
                          const float* S0, float* S_out, void* out, int B, int T, int Hk, int Hv, int KD, int VD,
                          bool l2norm, float eps, cudaStream_t stream);
// Optional gate inputs straight from the input projection (decode): a, b bf16 [B, Hv] with row strides lda, ldb,
// A_log and dt_bias fp32 [Hv]; the kernel then forms g = -exp(A_log) softplus(a + dt_bias) and beta = sigmoid(b)
// itself and ignores `g` / `beta`.
struct GdnRawGates {
  const __nv_bfloat16* a; long long lda;
  const __nv_bfloat16* b; long long ldb;
  const float* A_log; const float* dt_bias;
};
const char* gdn_decode_step(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv,
                            const float* g, const float* beta, float* S, int B, int Hk, int Hv, int KD, int VD,
                            bool l2norm, float eps, void* out, cudaStream_t stream, const GdnRawGates* raw_gates = nullptr);

// ---- chunked gated delta rule on tensor cores, forward and backward (csrc/kernels/gdn_tc.cu)
// All tensors fp32 and contiguous: q,k [B,T,Hk,128] (already L2-normalised, q scaled), v/out/dO/dq/dk/dv
// [B,T,Hv,128], g/beta/dG/dbeta [B,T,Hv]; per-chunk tensors (n = T / 64 chunks) Gc [B,Hv,n,64], gl [B,Hv,n],
// Tm [B,Hv,n,64,64], U/Wn/Kd/Vn/X0/dVn/dW [B,Hv,n,64,128], Sin/Y0/dSout [B,Hv,n,128,128], dGpart [2,B,T,Hv];
// states [B,Hv,128,128].
// T must be a multiple of 64 (at most 65536).  S0 and dS_final may be null.
const char* gdn_tc_forward(const float* q, const float* k, const float* v, const float* g, const float* beta, const float* S0,
                           int B, int T, int Hk, int Hv, float* Gc, float* gl, float* Tm, float* U, float* Wn, float* Kd,
                           float* out, float* S_out, float* Sin, float* Vn, cudaStream_t stream);
const char* gdn_tc_backward(const float* q, const float* k, const float* v, const float* beta, const float* Gc, const float* gl,
                            const float* Tm, const float* Wn, const float* Kd, const float* Vn, const float* Sin,
                            const float* dO, const float* dS_final, int B, int T, int Hk, int Hv, float* X0, float* Y0,
                            float* dVn, float* dSout, float* dW, float* dGpart, float* dq, float* dk, float* dv, float* dbeta,
                            float* dG, float* dS0, cudaStream_t stream);

// ---- expert parallelism over the symmetric heap (csrc/moe/ep.cu)
struct EpDispatchParams {
  const __nv_bfloat16* x; long long ldx;   // [T, H] rows to send
  const int* idx;                          // [T*k] global expert of every (token, slot) pair
  const float* pair_w;                     // optional per-pair scale applied while sending
  int T, k, H, E, E_local, rank, world;
  const int* my_counts;                    // [E] pairs per global expert on this rank
  PeerTable counts_all;                    // int [world][E] on every rank
  PeerTable xs;                            // bf16 [cap_rows][H] receive buffer on every rank
  PeerTable flags; unsigned epoch; unsigned long long limit_ns; int* status; int* abort_word;   // epoch: unused, the call number lives in `flags`
  int cap_rows;
  int* dest_row;                           // [T*k] row of each pair in its owner's buffer (out, or in when reuse_plan)
  int* tile_expert;                        // [cap_rows/128] local expert of each received tile, -1 unused (out)
  int* local_rows;                         // [1] padded rows in use on this rank (out)
  int reuse_plan;                          // 1: skip count exchange and planning (backward pass)
};
struct EpCombineParams {
  PeerTable ys;                            // bf16 [cap_rows][H] expert outputs on every rank
  const int* idx; const int* dest_row; const float* w;   // w optional [T*k]
  int T, k, H, E_local, rank, world;
  PeerTable flags; unsigned epoch; unsigned long long limit_ns; int* status; int* abort_word;
  __nv_bfloat16* out;                      // [T, H]
  __nv_bfloat16* keep_rows;                // optional [T*k, H]: the pulled rows, for the routing-weight gradient
};
const char* ep_dispatch(const EpDispatchParams& p, int num_sms, cudaStream_t stream);
const char* ep_combine(const EpCombineParams& p, int num_sms, cudaStream_t stream);

// ---- adapter gradients out[R, C] = U^T X (csrc/kernels/lora_grad.cu)
size_t lora_grad_workspace_floats(int R, int C, int n_splits);
int lora_grad_splits(int M, int C, int num_sms);
const char* lora_grad(const void* U, long long ldu, int R, const void* X, long long ldx, int C, int M, int n_splits,
                      float* partial, int* counters, float* out, long long ldo, cudaStream_t stream);

}  // namespace ferrl
