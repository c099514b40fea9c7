// torch op registration for the ferrl_b200 native library (namespace torch.ops.ferrl_b200).
// Thin argument checking + pointer extraction; all device work is in the .cu files.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "api.h"
#include "common.cuh"

namespace ferrl {
static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launch_count() { return g_launches.load(std::memory_order_relaxed); }
}  // namespace ferrl

namespace {

using at::Tensor;
using c10::optional;

#define FERRL_CHECK(err) do { const char* e__ = (err); TORCH_CHECK(e__ == nullptr, "ferrl_b200: ", e__); } while (0)

cudaStream_t stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

int dt(const Tensor& t) {
  if (t.scalar_type() == at::kBFloat16) return ferrl::kBF16;
  if (t.scalar_type() == at::kFloat) return ferrl::kF32;
  TORCH_CHECK(false, "ferrl_b200: tensors must be bfloat16 or float32, got ", t.scalar_type());
}

const void* optr(const optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

int num_sms() {
  static int n = 0;
  if (!n) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

// one status word per device, allocated once
int* status_word() {
  static std::mutex mu;
  static std::unordered_map<int, Tensor> words;
  std::lock_guard<std::mutex> g(mu);
  int dev = c10::cuda::current_device();
  auto it = words.find(dev);
  if (it == words.end())
    it = words.emplace(dev, at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, dev))).first;
  return it->second.data_ptr<int>();
}

// ---- canary mode (a test aid): every output the bindings allocate sits between two 512-byte pads filled with a
// pattern; check_canaries() counts pad bytes that changed since allocation, over all outputs made since the last
// check, and forgets them.  A kernel that stores outside its output is caught without any device-side tool.
std::atomic<bool> g_canary{false};
std::mutex g_canary_mu;
std::vector<std::pair<Tensor, int64_t>> g_canary_bufs;      // (raw byte buffer, payload bytes)
constexpr int64_t kCanaryPad = 512;
constexpr int kCanaryByte = 0xA5;

Tensor canary_alloc(at::IntArrayRef sizes, const at::TensorOptions& opt, bool zero) {
  int64_t numel = 1;
  for (auto d : sizes) numel *= d;
  const int64_t esz = static_cast<int64_t>(c10::elementSize(c10::typeMetaToScalarType(opt.dtype())));
  const int64_t nbytes = (numel * esz + 15) / 16 * 16;
  Tensor raw = at::empty({nbytes + 2 * kCanaryPad}, opt.dtype(at::kByte));
  raw.slice(0, 0, kCanaryPad).fill_(kCanaryByte);
  raw.slice(0, kCanaryPad + numel * esz, nbytes + 2 * kCanaryPad).fill_(kCanaryByte);
  Tensor out = raw.slice(0, kCanaryPad, kCanaryPad + numel * esz).view(c10::typeMetaToScalarType(opt.dtype())).view(sizes);
  if (zero) out.zero_();
  std::lock_guard<std::mutex> g(g_canary_mu);
  g_canary_bufs.emplace_back(raw, numel * esz);
  return out;
}
// not while a CUDA graph is being captured: the pad fills would only run at replay
bool canary_on() {
  if (!g_canary.load()) return false;
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  return cudaStreamIsCapturing(c10::cuda::getCurrentCUDAStream().stream(), &st) == cudaSuccess && st == cudaStreamCaptureStatusNone;
}
Tensor out_empty(at::IntArrayRef sizes, const at::TensorOptions& opt) {
  return canary_on() && opt.device().is_cuda() ? canary_alloc(sizes, opt, false) : at::empty(sizes, opt);
}
Tensor out_zeros(at::IntArrayRef sizes, const at::TensorOptions& opt) {
  return canary_on() && opt.device().is_cuda() ? canary_alloc(sizes, opt, true) : at::zeros(sizes, opt);
}
Tensor out_empty_like(const Tensor& t) {
  return canary_on() && t.is_cuda() && t.is_contiguous() ? canary_alloc(t.sizes(), t.options(), false) : at::empty_like(t);
}
void set_canary(bool on) { g_canary.store(on); }
int64_t check_canaries() {
  std::vector<std::pair<Tensor, int64_t>> bufs;
  {
    std::lock_guard<std::mutex> g(g_canary_mu);
    bufs.swap(g_canary_bufs);
  }
  int64_t bad = 0;
  for (auto& b : bufs) {
    const Tensor& raw = b.first;
    bad += raw.slice(0, 0, kCanaryPad).ne(kCanaryByte).sum().item<int64_t>();
    bad += raw.slice(0, kCanaryPad + b.second, raw.size(0)).ne(kCanaryByte).sum().item<int64_t>();
  }
  return bad;
}

ferrl::PeerTable table_of_fwd(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() <= ferrl::kMaxRanks, "too many ranks");
  ferrl::PeerTable t{};
  for (size_t i = 0; i < ptrs.size(); ++i) t.ptr[i] = reinterpret_cast<void*>(ptrs[i]);
  return t;
}

int64_t kernel_status() {
  int h = 0;
  C10_CUDA_CHECK(cudaMemcpy(&h, status_word(), sizeof(int), cudaMemcpyDeviceToHost));
  return h;
}
void reset_status() { C10_CUDA_CHECK(cudaMemsetAsync(status_word(), 0, sizeof(int), stream())); }

// Decode projections (M <= 128) with the activation tile resident in tensor memory
// (csrc/gemm/decode_gemm.cu).  Opt-in: measured inside a decode layer it is slower than the planner's
// choices (its per-tile exchange between the CTAs of a cluster takes about 2 us), so weights (static_b)
// take it only with FERRL_DECODE_GEMM=1 or set_decode_gemm(true).
bool g_decode_gemm = [] {
  const char* e = std::getenv("FERRL_DECODE_GEMM");
  return e && e[0] == '1';
}();
void set_decode_gemm(bool on) { g_decode_gemm = on; }

// glu_act: -1 none, 0 SiLU, 1 tanh-GELU (B rows interleaved in groups of 16: 8 gate rows, 8 up rows)
Tensor decode_gemm(const Tensor& A, const Tensor& B, const optional<Tensor>& residual, int64_t glu_act, int64_t max_clusters,
                   bool static_b, const optional<Tensor>& debug = optional<Tensor>()) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16 &&
                  A.dim() == 2 && B.dim() == 2 && A.size(1) == B.size(1) && A.stride(1) == 1 && B.stride(1) == 1,
              "decode_gemm: A [M,K], B [N,K] bf16, K-major");
  TORCH_CHECK(glu_act >= -1 && glu_act <= 1, "decode_gemm: glu_act -1, 0 or 1");
  const int M = A.size(0), N = B.size(0), K = A.size(1);
  TORCH_CHECK(ferrl::decode_gemm_supported(M, N, K, glu_act >= 0),
              "decode_gemm: needs 1 <= M <= 128, N a multiple of 64, K a multiple of 8 and >= 512 (no k groups with GLU)");
  c10::cuda::CUDAGuard guard(A.device());
  ferrl::DecodeGemmArgs a{};
  a.A = A.data_ptr(); a.B = B.data_ptr(); a.lda = A.stride(0); a.ldb = B.stride(0);
  a.M = M; a.N = N; a.K = K;
  Tensor out = out_empty({A.size(0), glu_act >= 0 ? B.size(0) / 2 : B.size(0)}, A.options());
  a.out = out.data_ptr(); a.ldo = out.stride(0);
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(glu_act < 0, "decode_gemm: no residual with the GLU epilogue");
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->dim() == 2 && residual->size(0) == M &&
                    residual->size(1) == N && residual->stride(1) == 1, "decode_gemm: residual bf16 [M,N]");
    a.residual = residual->data_ptr(); a.ldr = residual->stride(0);
  }
  a.glu_act = glu_act >= 0 ? static_cast<int>(glu_act) + 1 : 0;
  Tensor partial;
  const int groups = ferrl::decode_gemm_groups(K);
  if (groups > 1) {
    partial = out_empty({groups, A.size(0), B.size(0)}, A.options().dtype(at::kFloat));
    a.partial = partial.data_ptr<float>();
  }
  a.status = status_word();
  a.pdl = static_b ? 1 : 0;
  a.max_clusters = static_cast<int>(max_clusters);
  if (debug.has_value() && debug->defined()) {
    TORCH_CHECK(debug->scalar_type() == at::kLong && debug->numel() >= 64 && debug->is_cuda(), "decode_gemm: debug int64[64]");
    a.debug = reinterpret_cast<unsigned long long*>(debug->data_ptr<int64_t>());
  }
  FERRL_CHECK(ferrl::decode_gemm(a, stream()));
  return out;
}

// out[M,N] = A[M,K] B[N,K]^T (+ A2 B2^T) (+ residual)
Tensor gemm(const Tensor& A, const Tensor& B, const optional<Tensor>& A2, const optional<Tensor>& B2,
            const optional<Tensor>& residual, bool out_f32, int64_t force_bn, int64_t force_split, int64_t two_cta,
            const optional<Tensor>& debug, int64_t cluster_k, int64_t stream_k, bool static_b) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda(), "gemm: CUDA tensors required");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "gemm: operands must be bf16");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.size(1) == B.size(1), "gemm: A [M,K], B [N,K]");
  TORCH_CHECK(A.stride(1) == 1 && B.stride(1) == 1, "gemm: operands must be K-major");
  if (g_decode_gemm && static_b && !out_f32 && !(A2.has_value() && A2->defined()) && force_bn == 0 && force_split == 0 &&
      two_cta <= 0 && cluster_k == 0 && stream_k == 0 && B.size(0) <= 32768 &&
      ferrl::decode_gemm_supported(A.size(0), B.size(0), A.size(1), false))
    return decode_gemm(A, B, residual, -1, 0, true);
  c10::cuda::CUDAGuard guard(A.device());
  ferrl::GemmArgs a{};
  a.A = A.data_ptr(); a.B = B.data_ptr(); a.lda = A.stride(0); a.ldb = B.stride(0);
  a.M = A.size(0); a.N = B.size(0); a.K = A.size(1);
  if (A2.has_value() && A2->defined()) {
    TORCH_CHECK(B2.has_value() && B2->defined(), "gemm: A2 without B2");
    TORCH_CHECK(A2->scalar_type() == at::kBFloat16 && B2->scalar_type() == at::kBFloat16, "gemm: side operands bf16");
    TORCH_CHECK(A2->dim() == 2 && B2->dim() == 2 && A2->size(0) == a.M && B2->size(0) == a.N &&
                    A2->size(1) == B2->size(1) && A2->stride(1) == 1 && B2->stride(1) == 1,
                "gemm: side operand shapes");
    a.A2 = A2->data_ptr(); a.B2 = B2->data_ptr(); a.lda2 = A2->stride(0); a.ldb2 = B2->stride(0); a.K2 = A2->size(1);
  }
  Tensor out = out_empty({a.M, a.N}, A.options().dtype(out_f32 ? at::kFloat : at::kBFloat16));
  a.out = out.data_ptr(); a.ldo = a.N; a.out_f32 = out_f32;
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->dim() == 2 && residual->size(0) == a.M &&
                    residual->size(1) == a.N && residual->stride(1) == 1,
                "gemm: residual must be bf16 [M,N]");
    a.residual = residual->data_ptr(); a.ldr = residual->stride(0);
  }
  a.status = status_word(); a.num_sms = num_sms(); a.force_bn = static_cast<int>(force_bn);
  // static_b: B (and B2) are weights that no kernel earlier in the stream writes, so a decode-shaped
  // call may start streaming them before its predecessor has finished (programmatic dependent launch)
  a.pdl = (static_b && a.M <= 256) ? 1 : 0;
  if (two_cta > 0 && !out_f32) {   // forced
    TORCH_CHECK(two_cta == 128 || two_cta == 256, "gemm: two_cta must be 128 or 256");
    a.two_cta = static_cast<int>(two_cta);
    if (debug.has_value() && debug->defined()) a.debug = reinterpret_cast<unsigned int*>(debug->data_ptr<int>());
    FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
    return out;
  }
  int bn = 0, split = 1, cluster = 1;
  double est = 1e30;
  ferrl::gemm_plan(a.M, a.N, a.K, a.K2, a.num_sms, &bn, &split, &cluster, &est);
  {
    // stream-k: equal unit ranges per SM (csrc/gemm/tcgen05_gemm.cu); workspace and epochs live per device
    const bool eligible = a.M <= 128 && a.N >= 256 && (a.N % 4) == 0;
    bool use_sk = stream_k > 0 && eligible;
    if (stream_k == 0 && eligible && force_bn == 0 && force_split == 0 && cluster_k == 0 && two_cta == 0) {
      const long long kb = (a.K + 63) / 64 + (a.K2 + 63) / 64;
      const long long units = ((a.N + 255) / 256) * kb;
      const long long per = (units + a.num_sms - 1) / a.num_sms;
      const double t_sk = static_cast<double>(per) * (128 + 256) * 128.0 / 64e9 + 10e-6;
      use_sk = false && units >= a.num_sms && t_sk < est;   // measured slower than the planner's other choices: forced use only
    }
    TORCH_CHECK(stream_k <= 0 || eligible, "gemm: stream_k needs M <= 128, N >= 256, N % 4 == 0");
    if (use_sk) {
      static std::vector<Tensor> sk_ws(64), sk_flags(64);
      const int dev = A.get_device();
      const int max_ctas = 160;
      if (!sk_ws[dev].defined()) {
        sk_ws[dev] = out_empty({static_cast<long long>(max_ctas) * 2 * 128 * 256}, A.options().dtype(at::kFloat));
        sk_flags[dev] = out_zeros({max_ctas * 2 + 2}, A.options().dtype(at::kInt));   // flags, launch counter, done counter
      }
      a.stream_k = 1;
      a.sk_ws = sk_ws[dev].data_ptr<float>();
      a.sk_flags = reinterpret_cast<unsigned int*>(sk_flags[dev].data_ptr<int>());
      a.sk_max_ctas = max_ctas;
      if (debug.has_value() && debug->defined() && debug->scalar_type() == at::kLong && debug->numel() >= 4 * max_ctas)
        a.sk_debug = reinterpret_cast<unsigned long long*>(debug->data_ptr<int64_t>());
      FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
      return out;
    }
  }
  if (cluster_k > 1) {                      // forced cluster split: force_bn names the tile width
    TORCH_CHECK(force_bn > 0, "gemm: cluster_k needs force_bn");
    a.cluster_k = static_cast<int>(cluster_k);
    FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
    return out;
  }
  if (force_bn == 0 && force_split == 0 && cluster_k == 0 && cluster > 1) {
    a.force_bn = bn;
    a.cluster_k = cluster;
    FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
    return out;
  }
  if (force_bn == 0) a.force_bn = bn;
  if (force_split > 0) split = static_cast<int>(force_split);
  else if (force_bn != 0 || cluster > 1) split = 1;
  if (split <= 1 && force_bn == 0 && two_cta == 0 && !out_f32 && a.M >= 1024 && a.N >= 512) {
    // large problems: the two-SM kernel stages a third less per k-block and is not fill-bound
    a.two_cta = 256;
    FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
    return out;
  }
  Tensor partial;
  if (split > 1) {
    partial = out_empty({split, a.M, a.N}, A.options().dtype(at::kFloat));
    a.partial = partial.data_ptr<float>();
    a.split_k = split;
  }
  FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
  return out;
}

// act(x Wg^T) * (x Wu^T) in one kernel: W holds the gate and up rows interleaved in groups of 16
// (8 gate rows, then the 8 up rows of the same features); returns [M, N/2].
Tensor gemm_glu(const Tensor& A, const Tensor& B, int64_t act, bool static_b) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16 &&
                  A.dim() == 2 && B.dim() == 2 && A.size(1) == B.size(1) && A.stride(1) == 1 && B.stride(1) == 1,
              "gemm_glu: A [M,K], B [N,K] bf16, K-major");
  TORCH_CHECK((B.size(0) % 16) == 0 && (act == 0 || act == 1), "gemm_glu: N a multiple of 16, act 0 (silu) or 1 (tanh-gelu)");
  if (g_decode_gemm && static_b && ferrl::decode_gemm_supported(A.size(0), B.size(0), A.size(1), true))
    return decode_gemm(A, B, optional<Tensor>(), act, 0, true);
  c10::cuda::CUDAGuard guard(A.device());
  ferrl::GemmArgs a{};
  a.A = A.data_ptr(); a.B = B.data_ptr(); a.lda = A.stride(0); a.ldb = B.stride(0);
  a.M = A.size(0); a.N = B.size(0); a.K = A.size(1);
  Tensor out = out_empty({A.size(0), B.size(0) / 2}, A.options());
  a.out = out.data_ptr(); a.ldo = out.stride(0);
  a.status = status_word(); a.num_sms = num_sms();
  a.glu_act = static_cast<int>(act) + 1;
  a.pdl = (static_b && a.M <= 256) ? 1 : 0;
  int bn = 0, split = 1, cluster = 1;
  ferrl::gemm_plan(a.M, a.N, a.K, 0, a.num_sms, &bn, &split, &cluster, nullptr);
  if (split > 1 || cluster > 1 || bn == 32) bn = 128;      // the epilogue needs whole tiles in one CTA
  a.force_bn = bn;
  if (a.M == 0) return out;
  FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
  return out;
}

// Projection with an RMSNorm folded around it (decode chain).  `ss_in` [parts, M]: partial row sums of
// squares of A's rows; the rows of the result are scaled by rsqrt(sum / K + eps) (the norm weight must
// already be folded into B's columns).  `want_ss`: also return the partial row sums of squares of the
// stored output [parts', M] for the next projection.  glu_act: -1 none, 0 SiLU, 1 tanh-GELU (B interleaved).
std::tuple<Tensor, Tensor> gemm_norm(const Tensor& A, const Tensor& B, const optional<Tensor>& residual,
                                     const optional<Tensor>& ss_in, double eps, int64_t glu_act, bool want_ss, bool static_b) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16 &&
                  A.dim() == 2 && B.dim() == 2 && A.size(1) == B.size(1) && A.stride(1) == 1 && B.stride(1) == 1,
              "gemm_norm: A [M,K], B [N,K] bf16, K-major");
  TORCH_CHECK(glu_act >= -1 && glu_act <= 1 && (glu_act < 0 || (B.size(0) % 16) == 0), "gemm_norm: glu_act");
  TORCH_CHECK(glu_act < 0 || !(residual.has_value() && residual->defined()), "gemm_norm: no residual with the GLU epilogue");
  c10::cuda::CUDAGuard guard(A.device());
  ferrl::GemmArgs a{};
  a.A = A.data_ptr(); a.B = B.data_ptr(); a.lda = A.stride(0); a.ldb = B.stride(0);
  a.M = A.size(0); a.N = B.size(0); a.K = A.size(1);
  const int64_t n_out = glu_act >= 0 ? B.size(0) / 2 : B.size(0);
  Tensor out = out_empty({A.size(0), n_out}, A.options());
  a.out = out.data_ptr(); a.ldo = out.stride(0);
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->dim() == 2 && residual->size(0) == a.M &&
                    residual->size(1) == a.N && residual->stride(1) == 1, "gemm_norm: residual bf16 [M,N]");
    a.residual = residual->data_ptr(); a.ldr = residual->stride(0);
  }
  a.status = status_word(); a.num_sms = num_sms();
  a.glu_act = glu_act >= 0 ? static_cast<int>(glu_act) + 1 : 0;
  a.pdl = (static_b && a.M <= 256) ? 1 : 0;
  if (ss_in.has_value() && ss_in->defined()) {
    TORCH_CHECK(ss_in->scalar_type() == at::kFloat && ss_in->dim() == 2 && ss_in->is_contiguous() && ss_in->size(1) == a.M,
                "gemm_norm: ss_in float32 [parts, M]");
    a.ss_in = ss_in->data_ptr<float>(); a.ss_parts = ss_in->size(0); a.ss_ld = a.M;
    a.ss_inv_k = 1.0f / static_cast<float>(a.K); a.ss_eps = static_cast<float>(eps);
  }
  int bn = 0, split = 1, cluster = 1;
  ferrl::gemm_plan(a.M, a.N, a.K, 0, a.num_sms, &bn, &split, &cluster, nullptr);
  if (glu_act >= 0 || cluster <= 1) {
    if (split > 1 || cluster > 1 || bn == 32) bn = 128;      // whole tiles in one CTA
    cluster = 1;
  }
  a.force_bn = bn;
  a.cluster_k = cluster > 1 ? cluster : 0;
  Tensor ss_out;
  if (want_ss) {
    TORCH_CHECK(glu_act < 0, "gemm_norm: no row statistics behind the GLU epilogue");
    ss_out = out_empty({ferrl::gemm_ss_parts(a.N, bn, cluster), static_cast<long long>(a.M)}, A.options().dtype(at::kFloat));
    a.ss_out = ss_out.data_ptr<float>(); a.ss_ld = a.M;
  } else {
    ss_out = out_empty({0}, A.options().dtype(at::kFloat));
  }
  if (a.M == 0) return {out, ss_out};
  FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
  return {out, ss_out};
}

Tensor row_sumsq(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "row_sumsq: bf16 [M,H]");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor ss = out_empty({1, x.size(0)}, x.options().dtype(at::kFloat));
  FERRL_CHECK(ferrl::row_sumsq(x.data_ptr(), x.stride(0), ss.data_ptr<float>(), x.size(0), x.size(1), stream()));
  return ss;
}

// Row-parallel projection fused with its tensor-parallel all-reduce:
// out = sum_over_ranks(A_r B_r^T (+ A2 B2^T)) (+ residual), identical on every rank.
Tensor gemm_allreduce(const Tensor& A, const Tensor& B, const optional<Tensor>& A2, const optional<Tensor>& B2,
                      const optional<Tensor>& residual, std::vector<int64_t> stage, std::vector<int64_t> outbuf,
                      std::vector<int64_t> flags, int64_t rank, int64_t world, int64_t epoch, int64_t max_tiles,
                      int64_t stage_elems, int64_t out_elems, double limit_s, const optional<Tensor>& debug, int64_t mc_stage,
                      int64_t mc_outbuf, bool scatter) {
  TORCH_CHECK(A.is_cuda() && A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16, "gemm_allreduce: bf16");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.size(1) == B.size(1) && A.stride(1) == 1 && B.stride(1) == 1, "gemm_allreduce: shapes");
  c10::cuda::CUDAGuard guard(A.device());
  ferrl::GemmArgs a{};
  a.A = A.data_ptr(); a.B = B.data_ptr(); a.lda = A.stride(0); a.ldb = B.stride(0);
  a.M = A.size(0); a.N = B.size(0); a.K = A.size(1);
  if (A2.has_value() && A2->defined()) {
    TORCH_CHECK(B2.has_value() && B2->defined() && A2->stride(1) == 1 && B2->stride(1) == 1, "gemm_allreduce: side operands");
    a.A2 = A2->data_ptr(); a.B2 = B2->data_ptr(); a.lda2 = A2->stride(0); a.ldb2 = B2->stride(0); a.K2 = A2->size(1);
  }
  // reduce-scatter form: this rank's M / world rows of the sum
  TORCH_CHECK(!scatter || (world > 1 && a.M % (world * 128) == 0), "gemm_allreduce: the reduce-scatter form needs rows % (world x 128) == 0");
  Tensor out = out_empty({scatter ? a.M / world : a.M, a.N}, A.options());
  a.ar_scatter = scatter ? 1 : 0;
  a.out = out.data_ptr(); a.ldo = a.N; a.out_f32 = false;
  if (residual.has_value() && residual->defined()) { a.residual = residual->data_ptr(); a.ldr = residual->stride(0); }
  a.status = status_word(); a.num_sms = num_sms();
  a.force_bn = (a.N >= 256 && static_cast<int64_t>((a.M + 127) / 128) * ((a.N + 255) / 256) >= num_sms()) ? 256 : 128;
  if (a.N < 128) a.force_bn = 64;
  a.ar_world = world; a.ar_rank = rank; (void)epoch; a.ar_max_tiles = max_tiles;   // the call number lives on the device
  a.ar_limit_ns = static_cast<unsigned long long>(limit_s * 1e9);
  a.ar_stage_elems = stage_elems; a.ar_out_elems = out_elems;
  if (debug.has_value() && debug->defined() && debug->scalar_type() == at::kLong && debug->numel() >= 160 * 16 * 4)
    a.ar_debug = reinterpret_cast<unsigned long long*>(debug->data_ptr<int64_t>());
  a.ar_stage = table_of_fwd(stage); a.ar_outbuf = table_of_fwd(outbuf); a.ar_flags = table_of_fwd(flags);
  a.ar_mc_stage = reinterpret_cast<void*>(mc_stage); a.ar_mc_outbuf = reinterpret_cast<void*>(mc_outbuf);
  FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
  return out;
}

// Column-parallel projection fused with the all-gather of its sequence-sharded input: `src` are every rank's gather
// buffers ([M, K] bf16, packed; this rank has filled its own M / world rows of src[rank]); out = gathered A B^T (+ A2 B2^T).
// After the call src[rank] holds all M rows.
Tensor gemm_allgather(const Tensor& B, const optional<Tensor>& A2, const optional<Tensor>& B2, std::vector<int64_t> src,
                      std::vector<int64_t> flags, int64_t rank, int64_t world, int64_t max_tiles, int64_t M, int64_t K,
                      double limit_s) {
  TORCH_CHECK(B.is_cuda() && B.scalar_type() == at::kBFloat16 && B.dim() == 2 && B.size(1) == K && B.stride(1) == 1, "gemm_allgather: B bf16 [N, K]");
  TORCH_CHECK(world > 1 && M % (world * 128) == 0 && K % 8 == 0, "gemm_allgather: rows % (world x 128) == 0 and K % 8 == 0");
  c10::cuda::CUDAGuard guard(B.device());
  ferrl::GemmArgs a{};
  a.ag_src = table_of_fwd(src);
  a.A = a.ag_src.ptr[rank]; a.B = B.data_ptr(); a.lda = K; a.ldb = B.stride(0);
  a.M = M; a.N = B.size(0); a.K = K;
  if (A2.has_value() && A2->defined()) {
    TORCH_CHECK(B2.has_value() && B2->defined() && A2->stride(1) == 1 && B2->stride(1) == 1 && A2->size(0) == M &&
                    A2->scalar_type() == at::kBFloat16 && B2->scalar_type() == at::kBFloat16, "gemm_allgather: side operands");
    a.A2 = A2->data_ptr(); a.B2 = B2->data_ptr(); a.lda2 = A2->stride(0); a.ldb2 = B2->stride(0); a.K2 = A2->size(1);
  }
  Tensor out = out_empty({a.M, a.N}, B.options());
  a.out = out.data_ptr(); a.ldo = a.N; a.out_f32 = false;
  a.status = status_word(); a.num_sms = num_sms();
  a.force_bn = (a.N >= 256 && static_cast<int64_t>((a.M + 127) / 128) * ((a.N + 255) / 256) >= num_sms()) ? 256 : 128;
  if (a.N < 128) a.force_bn = 64;
  a.ar_world = world; a.ar_rank = rank; a.ar_max_tiles = max_tiles; a.ar_gather = 1;
  a.ar_limit_ns = static_cast<unsigned long long>(limit_s * 1e9);
  a.ar_flags = table_of_fwd(flags);
  FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
  return out;
}

// out[R, C] = U^T X, U [M, R] and X [M, C] bf16 (row strides free, last dim contiguous), fp32 result
Tensor lora_grad(const Tensor& U, const Tensor& X) {
  TORCH_CHECK(U.is_cuda() && U.scalar_type() == at::kBFloat16 && X.scalar_type() == at::kBFloat16 && U.dim() == 2 &&
                  X.dim() == 2 && U.size(0) == X.size(0) && U.stride(1) == 1 && X.stride(1) == 1, "lora_grad: U [M,R], X [M,C] bf16");
  c10::cuda::CUDAGuard guard(U.device());
  const int64_t M = U.size(0), R = U.size(1), C = X.size(1);
  Tensor out = out_empty({R, C}, U.options().dtype(at::kFloat));
  if (M == 0) return out.zero_();
  const int splits = ferrl::lora_grad_splits(M, C, num_sms());
  Tensor partial = out_empty({static_cast<long long>(ferrl::lora_grad_workspace_floats(R, C, splits))}, out.options());
  // per-device counters, zero between calls (the kernel resets the ones it used)
  static std::vector<Tensor> counters(64);
  const int dev = U.get_device();
  const int64_t tiles = (C + 127) / 128;
  if (!counters[dev].defined() || counters[dev].numel() < tiles)
    counters[dev] = out_zeros({std::max<int64_t>(tiles, 4096)}, U.options().dtype(at::kInt));
  FERRL_CHECK(ferrl::lora_grad(U.data_ptr(), U.stride(0), R, X.data_ptr(), X.stride(0), C, M, splits,
                               partial.data_ptr<float>(), counters[dev].data_ptr<int>(), out.data_ptr<float>(), C, stream()));
  return out;
}

// ---------------------------------------------------------------- GatedDeltaNet
// x [B, L, C] bf16 (last dim contiguous, rows evenly strided), w [C, K], left [B, C, K-1] or none -> y [B, L, C]
Tensor gdn_conv_fwd(const Tensor& x, const Tensor& w, const optional<Tensor>& left, bool act) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 3 && x.stride(2) == 1 &&
                  x.stride(0) == x.size(1) * x.stride(1), "gdn_conv_fwd: x bf16 [B,L,C] with uniform row stride");
  TORCH_CHECK(w.scalar_type() == at::kBFloat16 && w.is_contiguous() && w.size(0) == x.size(2), "gdn_conv_fwd: w bf16 [C,K]");
  c10::cuda::CUDAGuard guard(x.device());
  const void* lp = nullptr;
  if (left.has_value() && left->defined()) {
    TORCH_CHECK(left->scalar_type() == at::kBFloat16 && left->is_contiguous() && left->size(0) == x.size(0) &&
                    left->size(1) == x.size(2) && left->size(2) == w.size(1) - 1, "gdn_conv_fwd: left bf16 [B,C,K-1]");
    lp = left->data_ptr();
  }
  Tensor y = out_empty({x.size(0), x.size(1), x.size(2)}, x.options());
  FERRL_CHECK(ferrl::gdn_conv_fwd(x.data_ptr(), x.stride(1), w.data_ptr(), lp, x.size(0), x.size(1), x.size(2), w.size(1),
                                  act, y.data_ptr(), stream()));
  return y;
}

Tensor gdn_conv_bwd(const Tensor& x, const Tensor& w, const optional<Tensor>& left, const Tensor& dy, bool act) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 3 && x.stride(2) == 1 &&
                  x.stride(0) == x.size(1) * x.stride(1) && dy.is_contiguous() && dy.scalar_type() == at::kBFloat16,
              "gdn_conv_bwd: shapes");
  c10::cuda::CUDAGuard guard(x.device());
  const void* lp = (left.has_value() && left->defined()) ? left->data_ptr() : nullptr;
  Tensor dx = out_empty({x.size(0), x.size(1), x.size(2)}, x.options());
  FERRL_CHECK(ferrl::gdn_conv_bwd(x.data_ptr(), x.stride(1), w.data_ptr(), lp, dy.data_ptr(), x.size(0), x.size(1),
                                  x.size(2), w.size(1), act, dx.data_ptr(), stream()));
  return dx;
}

// one token: x [B, C] (row stride free), state [B, C, K-1] updated in place -> y [B, C]
Tensor gdn_conv_step(const Tensor& x, const Tensor& w, Tensor state, bool act) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "gdn_conv_step: x bf16 [B,C]");
  TORCH_CHECK(state.scalar_type() == at::kBFloat16 && state.is_contiguous() && state.size(0) == x.size(0) &&
                  state.size(1) == x.size(1) && state.size(2) == w.size(1) - 1 && w.is_contiguous(), "gdn_conv_step: state bf16 [B,C,K-1]");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = out_empty({x.size(0), x.size(1)}, x.options());
  FERRL_CHECK(ferrl::gdn_conv_step(x.data_ptr(), x.stride(0), w.data_ptr(), state.data_ptr(), x.size(0), x.size(1),
                                   w.size(1), act, y.data_ptr(), stream()));
  return y;
}

// q,k [B, Hk*KD], v [B, Hv*VD] bf16 (row strides free), g,beta [B,Hv] f32, S [B,Hv,KD,VD] f32 in place -> o [B,Hv,VD]
Tensor gdn_decode_step(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta, Tensor S,
                       bool l2norm, double eps) {
  TORCH_CHECK(S.is_cuda() && S.scalar_type() == at::kFloat && S.dim() == 4 && S.is_contiguous(), "gdn_decode_step: S f32 [B,Hv,KD,VD]");
  const int64_t B = S.size(0), Hv = S.size(1), KD = S.size(2), VD = S.size(3);
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16 &&
                  q.dim() == 2 && k.dim() == 2 && v.dim() == 2 && q.stride(1) == 1 && k.stride(1) == 1 && v.stride(1) == 1 &&
                  q.size(0) == B && v.size(1) == Hv * VD && q.size(1) % KD == 0 && k.size(1) == q.size(1),
              "gdn_decode_step: q,k [B,Hk*KD], v [B,Hv*VD] bf16");
  TORCH_CHECK(g.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat && g.is_contiguous() && beta.is_contiguous() &&
                  g.numel() == B * Hv && beta.numel() == B * Hv, "gdn_decode_step: g,beta f32 [B,Hv]");
  c10::cuda::CUDAGuard guard(S.device());
  Tensor out = out_empty({B, Hv, VD}, q.options());
  FERRL_CHECK(ferrl::gdn_decode_step(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0),
                                     g.data_ptr<float>(), beta.data_ptr<float>(), S.data_ptr<float>(), B, q.size(1) / KD,
                                     Hv, KD, VD, l2norm, static_cast<float>(eps), out.data_ptr(), stream()));
  return out;
}

// Same step with the gates taken from the input projection: a, b bf16 [B, Hv] (row strides free), A_log and
// dt_bias f32 [Hv]; g and beta are formed inside the kernel.
Tensor gdn_decode_step_raw(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& a, const Tensor& b,
                           const Tensor& A_log, const Tensor& dt_bias, Tensor S, bool l2norm, double eps) {
  TORCH_CHECK(S.is_cuda() && S.scalar_type() == at::kFloat && S.dim() == 4 && S.is_contiguous(), "gdn_decode_step_raw: S f32 [B,Hv,KD,VD]");
  const int64_t B = S.size(0), Hv = S.size(1), KD = S.size(2), VD = S.size(3);
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16 &&
                  q.dim() == 2 && k.dim() == 2 && v.dim() == 2 && q.stride(1) == 1 && k.stride(1) == 1 && v.stride(1) == 1 &&
                  q.size(0) == B && v.size(1) == Hv * VD && q.size(1) % KD == 0 && k.size(1) == q.size(1),
              "gdn_decode_step_raw: q,k [B,Hk*KD], v [B,Hv*VD] bf16");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.dim() == 2 && b.dim() == 2 &&
                  a.size(0) == B && b.size(0) == B && a.size(1) == Hv && b.size(1) == Hv && a.stride(1) == 1 && b.stride(1) == 1,
              "gdn_decode_step_raw: a,b bf16 [B,Hv]");
  TORCH_CHECK(A_log.scalar_type() == at::kFloat && dt_bias.scalar_type() == at::kFloat && A_log.is_contiguous() &&
                  dt_bias.is_contiguous() && A_log.numel() == Hv && dt_bias.numel() == Hv, "gdn_decode_step_raw: A_log, dt_bias f32 [Hv]");
  c10::cuda::CUDAGuard guard(S.device());
  Tensor out = out_empty({B, Hv, VD}, q.options());
  ferrl::GdnRawGates raw{reinterpret_cast<const __nv_bfloat16*>(a.data_ptr()), a.stride(0),
                         reinterpret_cast<const __nv_bfloat16*>(b.data_ptr()), b.stride(0), A_log.data_ptr<float>(),
                         dt_bias.data_ptr<float>()};
  FERRL_CHECK(ferrl::gdn_decode_step(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0), nullptr,
                                     nullptr, S.data_ptr<float>(), B, q.size(1) / KD, Hv, KD, VD, l2norm, static_cast<float>(eps),
                                     out.data_ptr(), stream(), &raw));
  return out;
}

// q,k [B,T,Hk,KD], v [B,T,Hv,VD] bf16 (head dims contiguous, token/batch strides free), g,beta [B,T,Hv] f32,
// S0 [B,Hv,KD,VD] f32 or none -> (out [B,T,Hv,VD] bf16, S [B,Hv,KD,VD] f32)
static void gdn_tc_check(const Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), "gdn_tc: ", what, " must be contiguous fp32 on the GPU");
}

// Tensor-core chunked gated delta rule. Returns (out, S_final, Gc, gl, Tm, Wn, Kd, Vn, Sin); everything after
// S_final feeds gdn_tc_bwd.
std::vector<Tensor> gdn_tc_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g, const Tensor& beta,
                               const optional<Tensor>& S0) {
  gdn_tc_check(q, "q"); gdn_tc_check(k, "k"); gdn_tc_check(v, "v"); gdn_tc_check(g, "g"); gdn_tc_check(beta, "beta");
  TORCH_CHECK(q.dim() == 4 && k.sizes() == q.sizes() && v.dim() == 4 && q.size(3) == 128 && v.size(3) == 128 &&
                  v.size(0) == q.size(0) && v.size(1) == q.size(1), "gdn_tc_fwd: q,k [B,T,Hk,128], v [B,T,Hv,128]");
  const int64_t B = q.size(0), T = q.size(1), Hk = q.size(2), Hv = v.size(2);
  TORCH_CHECK(T % 64 == 0 && Hv % Hk == 0, "gdn_tc_fwd: T must be a multiple of 64 and Hv a multiple of Hk");
  TORCH_CHECK(g.numel() == B * T * Hv && beta.numel() == B * T * Hv, "gdn_tc_fwd: g,beta [B,T,Hv]");
  const float* s0 = nullptr;
  if (S0.has_value()) {
    gdn_tc_check(*S0, "S0");
    TORCH_CHECK(S0->numel() == B * Hv * 128 * 128, "gdn_tc_fwd: S0 [B,Hv,128,128]");
    s0 = S0->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t n = T / 64;
  auto opt = q.options();
  Tensor out = out_empty({B, T, Hv, 128}, opt), S_out = out_empty({B, Hv, 128, 128}, opt);
  Tensor Gc = out_empty({B, Hv, n, 64}, opt), gl = out_empty({B, Hv, n}, opt), Tm = out_empty({B, Hv, n, 64, 64}, opt);
  Tensor U = out_empty({B, Hv, n, 64, 128}, opt), Wn = out_empty({B, Hv, n, 64, 128}, opt), Kd = out_empty({B, Hv, n, 64, 128}, opt);
  Tensor Vn = out_empty({B, Hv, n, 64, 128}, opt), Sin = out_empty({B, Hv, n, 128, 128}, opt);
  FERRL_CHECK(ferrl::gdn_tc_forward(q.data_ptr<float>(), k.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(),
                                    beta.data_ptr<float>(), s0, B, T, Hk, Hv, Gc.data_ptr<float>(), gl.data_ptr<float>(),
                                    Tm.data_ptr<float>(), U.data_ptr<float>(), Wn.data_ptr<float>(), Kd.data_ptr<float>(),
                                    out.data_ptr<float>(), S_out.data_ptr<float>(), Sin.data_ptr<float>(), Vn.data_ptr<float>(),
                                    stream()));
  return {out, S_out, Gc, gl, Tm, Wn, Kd, Vn, Sin};
}

// Returns (dq [B,T,Hv,128] per value head, dk likewise, dv, dbeta, dG, dS0); dG is the gradient of the
// in-chunk cumulative log decay (the caller's reverse cumulative sum inside each chunk gives dg).
std::vector<Tensor> gdn_tc_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& beta, const Tensor& Gc,
                               const Tensor& gl, const Tensor& Tm, const Tensor& Wn, const Tensor& Kd, const Tensor& Vn,
                               const Tensor& Sin, const Tensor& dO, const optional<Tensor>& dS_final) {
  gdn_tc_check(q, "q"); gdn_tc_check(k, "k"); gdn_tc_check(v, "v"); gdn_tc_check(beta, "beta"); gdn_tc_check(Gc, "Gc");
  gdn_tc_check(gl, "gl"); gdn_tc_check(Tm, "Tm"); gdn_tc_check(Wn, "Wn"); gdn_tc_check(Kd, "Kd"); gdn_tc_check(Vn, "Vn");
  gdn_tc_check(Sin, "Sin"); gdn_tc_check(dO, "dO");
  const int64_t B = q.size(0), T = q.size(1), Hk = q.size(2), Hv = v.size(2), n = T / 64;
  TORCH_CHECK(T % 64 == 0 && dO.sizes() == v.sizes() && Vn.numel() == B * Hv * n * 64 * 128 &&
                  Sin.numel() == B * Hv * n * 128 * 128 && Tm.numel() == B * Hv * n * 64 * 64 && Wn.numel() == Vn.numel() &&
                  Kd.numel() == Vn.numel() && Gc.numel() == B * Hv * n * 64 && gl.numel() == B * Hv * n &&
                  beta.numel() == B * T * Hv,
              "gdn_tc_bwd: saved tensors do not match the inputs");
  const float* dsf = nullptr;
  if (dS_final.has_value()) {
    gdn_tc_check(*dS_final, "dS_final");
    TORCH_CHECK(dS_final->numel() == B * Hv * 128 * 128, "gdn_tc_bwd: dS_final [B,Hv,128,128]");
    dsf = dS_final->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(q.device());
  auto opt = q.options();
  Tensor X0 = out_empty_like(Vn), Y0 = out_empty_like(Sin), dVn = out_empty_like(Vn), dSout = out_empty_like(Sin);
  Tensor dW = out_empty_like(Vn), dGpart = out_empty({2, B, T, Hv}, opt);
  Tensor dq = out_empty({B, T, Hv, 128}, opt), dk = out_empty({B, T, Hv, 128}, opt), dv = out_empty_like(v);
  Tensor dbeta = out_empty({B, T, Hv}, opt), dG = out_empty({B, T, Hv}, opt), dS0 = out_empty({B, Hv, 128, 128}, opt);
  FERRL_CHECK(ferrl::gdn_tc_backward(q.data_ptr<float>(), k.data_ptr<float>(), v.data_ptr<float>(), beta.data_ptr<float>(),
                                     Gc.data_ptr<float>(), gl.data_ptr<float>(), Tm.data_ptr<float>(), Wn.data_ptr<float>(),
                                     Kd.data_ptr<float>(), Vn.data_ptr<float>(), Sin.data_ptr<float>(), dO.data_ptr<float>(), dsf,
                                     B, T, Hk, Hv, X0.data_ptr<float>(), Y0.data_ptr<float>(), dVn.data_ptr<float>(),
                                     dSout.data_ptr<float>(), dW.data_ptr<float>(), dGpart.data_ptr<float>(), dq.data_ptr<float>(),
                                     dk.data_ptr<float>(), dv.data_ptr<float>(),
                                     dbeta.data_ptr<float>(), dG.data_ptr<float>(), dS0.data_ptr<float>(), stream()));
  return {dq, dk, dv, dbeta, dG, dS0};
}

std::tuple<Tensor, Tensor> gdn_chunk_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& g,
                                         const Tensor& beta, const optional<Tensor>& S0, bool l2norm, double eps) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
                  v.scalar_type() == at::kBFloat16 && q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "gdn_chunk_fwd: bf16 [B,T,H,D]");
  const int64_t B = q.size(0), T = q.size(1), Hk = q.size(2), KD = q.size(3), Hv = v.size(2), VD = v.size(3);
  auto packed = [](const Tensor& t) { return t.stride(3) == 1 && t.stride(2) == t.size(3); };
  TORCH_CHECK(packed(q) && packed(k) && packed(v), "gdn_chunk_fwd: heads must be packed in the last two dims");
  TORCH_CHECK(g.scalar_type() == at::kFloat && beta.scalar_type() == at::kFloat && g.is_contiguous() && beta.is_contiguous() &&
                  g.numel() == B * T * Hv && beta.numel() == B * T * Hv, "gdn_chunk_fwd: g,beta f32 [B,T,Hv]");
  c10::cuda::CUDAGuard guard(q.device());
  const float* s0 = nullptr;
  Tensor s0c;
  if (S0.has_value() && S0->defined()) {
    s0c = S0->to(at::kFloat).contiguous();
    TORCH_CHECK(s0c.numel() == B * Hv * KD * VD, "gdn_chunk_fwd: state [B,Hv,KD,VD]");
    s0 = s0c.data_ptr<float>();
  }
  Tensor out = out_empty({B, T, Hv, VD}, q.options());
  Tensor S = out_empty({B, Hv, KD, VD}, q.options().dtype(at::kFloat));
  FERRL_CHECK(ferrl::gdn_chunk_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), q.stride(1), k.stride(0),
                                   k.stride(1), v.stride(0), v.stride(1), g.data_ptr<float>(), beta.data_ptr<float>(), s0,
                                   S.data_ptr<float>(), out.data_ptr(), B, T, Hk, Hv, KD, VD, l2norm,
                                   static_cast<float>(eps), stream()));
  return {out, S};
}

// ---------------------------------------------------------------- mixture of experts
// logits [T, E] fp32 -> (probs [T,E] f32, scores [T,k] f32, idx [T,k] i32, counts [E] i32)
std::tuple<Tensor, Tensor, Tensor, Tensor> moe_route(const Tensor& logits, int64_t k, bool renorm) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1, "moe_route: fp32 [T,E]");
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0), E = logits.size(1);
  Tensor probs = out_empty({T, E}, logits.options());
  Tensor scores = out_empty({T, k}, logits.options());
  Tensor idx = out_empty({T, k}, logits.options().dtype(at::kInt));
  Tensor counts = out_empty({E}, logits.options().dtype(at::kInt));
  FERRL_CHECK(ferrl::moe_route(logits.data_ptr<float>(), logits.stride(0), T, E, k, renorm, probs.data_ptr<float>(),
                               scores.data_ptr<float>(), idx.data_ptr<int>(), counts.data_ptr<int>(), stream()));
  return {probs, scores, idx, counts};
}

// idx [T,k] i32, counts [E] -> (row_of [T*k], token_of [max_rows], tile_expert [max_rows/128], seg_start [E+1])
std::tuple<Tensor, Tensor, Tensor, Tensor> moe_plan(const Tensor& idx, const Tensor& counts) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kInt && idx.dim() == 2 && idx.is_contiguous(), "moe_plan: idx i32 [T,k]");
  c10::cuda::CUDAGuard guard(idx.device());
  const int64_t T = idx.size(0), k = idx.size(1), E = counts.size(0);
  const int64_t pairs = T * k;
  // every expert may waste up to 127 rows of padding, but never more rows than tiles it could fill
  const int64_t max_rows = (pairs + std::min<int64_t>(E, pairs) * 127 + 127) / 128 * 128;
  auto io = idx.options();
  Tensor row_of = out_empty({pairs}, io);
  Tensor token_of = at::full({std::max<int64_t>(max_rows, 128)}, -1, io);
  Tensor tile_expert = at::full({std::max<int64_t>(max_rows / 128, 1)}, -1, io);
  Tensor seg_start = out_zeros({E + 1}, io);
  FERRL_CHECK(ferrl::moe_plan(idx.data_ptr<int>(), counts.data_ptr<int>(), pairs, k, E, max_rows, row_of.data_ptr<int>(),
                              token_of.data_ptr<int>(), tile_expert.data_ptr<int>(), seg_start.data_ptr<int>(), stream()));
  return {row_of, token_of, tile_expert, seg_start};
}

// xs[row] = (pair_w ? pair_w[pair of row] : 1) * x[token_of[row]]; padding rows are zero
Tensor moe_gather(const Tensor& x, const Tensor& token_of, const optional<Tensor>& pair_w, const Tensor& row_of) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "moe_gather: bf16 [T,H]");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = token_of.size(0), H = x.size(1);
  Tensor xs = out_empty({rows, H}, x.options());
  Tensor row_scale;
  const float* pw = nullptr;
  if (pair_w.has_value() && pair_w->defined()) {
    TORCH_CHECK(pair_w->scalar_type() == at::kFloat && pair_w->is_contiguous() && pair_w->numel() == row_of.numel(), "moe_gather: pair weights f32 [T*k]");
    row_scale = out_zeros({rows}, x.options().dtype(at::kFloat));
    pw = pair_w->data_ptr<float>();
  }
  FERRL_CHECK(ferrl::moe_gather(x.data_ptr(), x.stride(0), token_of.data_ptr<int>(), pw, row_of.data_ptr<int>(),
                                row_of.numel(), pw ? row_scale.data_ptr<float>() : nullptr, rows, H, xs.data_ptr(), stream()));
  return xs;
}

// ys[rows, N] = xs[rows, K] x W[e(row)]^T with W [E, N, K]; rows sorted by expert in 128-row segments
Tensor moe_grouped_gemm(const Tensor& xs, const Tensor& W, const Tensor& tile_expert, const optional<Tensor>& out_buf) {
  TORCH_CHECK(xs.is_cuda() && xs.scalar_type() == at::kBFloat16 && W.scalar_type() == at::kBFloat16, "moe_grouped_gemm: bf16");
  TORCH_CHECK(xs.dim() == 2 && W.dim() == 3 && W.is_contiguous() && xs.is_contiguous() && xs.size(1) == W.size(2), "moe_grouped_gemm: xs [R,K], W [E,N,K]");
  TORCH_CHECK(xs.size(0) % 128 == 0 && tile_expert.numel() * 128 >= xs.size(0) && tile_expert.scalar_type() == at::kInt, "moe_grouped_gemm: rows in 128-row tiles with one expert id each");
  c10::cuda::CUDAGuard guard(xs.device());
  ferrl::GemmArgs a{};
  a.A = xs.data_ptr(); a.B = W.data_ptr(); a.lda = xs.stride(0); a.ldb = W.size(2);
  a.M = xs.size(0); a.N = W.size(1); a.K = xs.size(1);
  a.tile_expert = tile_expert.data_ptr<int>(); a.n_experts = W.size(0);
  // rows of unused tiles are never written: start from zeros so padding stays finite downstream
  Tensor out;
  if (out_buf.has_value() && out_buf->defined()) {
    TORCH_CHECK(out_buf->scalar_type() == at::kBFloat16 && out_buf->is_contiguous() && out_buf->dim() == 2 &&
                    out_buf->size(0) == a.M && out_buf->size(1) == a.N, "moe_grouped_gemm: out buffer bf16 [R,N]");
    out = *out_buf;
  } else {
    out = out_zeros({a.M, a.N}, xs.options());
  }
  a.out = out.data_ptr(); a.ldo = a.N;
  a.status = status_word(); a.num_sms = num_sms();
  a.force_bn = a.N >= 256 ? 256 : (a.N >= 128 ? 128 : 64);
  FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
  return out;
}

// Expert-parallel dispatch: see csrc/moe/ep.cu.  dest_row / tile_expert / local_rows are outputs
// unless reuse_plan (then dest_row is the forward plan).
void ep_dispatch(const Tensor& x, const Tensor& idx, const optional<Tensor>& pair_w, const Tensor& counts,
                 std::vector<int64_t> counts_all, std::vector<int64_t> xs, std::vector<int64_t> flags, int64_t rank,
                 int64_t world, int64_t epoch, double limit_s, int64_t cap_rows, Tensor dest_row, Tensor tile_expert,
                 Tensor local_rows, bool reuse_plan, Tensor abort_word) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "ep_dispatch: x bf16 [T,H]");
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.dim() == 2 && idx.is_contiguous() && idx.size(0) == x.size(0), "ep_dispatch: idx i32 [T,k]");
  TORCH_CHECK(counts.scalar_type() == at::kInt && counts.is_contiguous(), "ep_dispatch: counts i32 [E]");
  TORCH_CHECK(dest_row.scalar_type() == at::kInt && dest_row.numel() == idx.numel() && tile_expert.numel() * 128 >= cap_rows, "ep_dispatch: plan buffers");
  c10::cuda::CUDAGuard guard(x.device());
  ferrl::EpDispatchParams p{};
  p.x = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()); p.ldx = x.stride(0);
  p.idx = idx.data_ptr<int>();
  if (pair_w.has_value() && pair_w->defined()) {
    TORCH_CHECK(pair_w->scalar_type() == at::kFloat && pair_w->is_contiguous() && pair_w->numel() == idx.numel(), "ep_dispatch: pair weights");
    p.pair_w = pair_w->data_ptr<float>();
  }
  p.T = x.size(0); p.k = idx.size(1); p.H = x.size(1); p.E = counts.numel(); p.E_local = p.E / world;
  p.rank = rank; p.world = world; p.my_counts = counts.data_ptr<int>();
  p.counts_all = table_of_fwd(counts_all); p.xs = table_of_fwd(xs); p.flags = table_of_fwd(flags);
  p.epoch = static_cast<unsigned>(epoch); p.limit_ns = static_cast<unsigned long long>(limit_s * 1e9);
  p.status = status_word(); p.abort_word = abort_word.data_ptr<int>(); p.cap_rows = cap_rows;
  p.dest_row = dest_row.data_ptr<int>(); p.tile_expert = tile_expert.data_ptr<int>(); p.local_rows = local_rows.data_ptr<int>();
  p.reuse_plan = reuse_plan ? 1 : 0;
  FERRL_CHECK(ferrl::ep_dispatch(p, num_sms(), stream()));
}

// Expert-parallel combine: out[t] = sum_j w[t,j] * ys[owner(t,j)][dest_row[t,j]]
Tensor ep_combine(std::vector<int64_t> ys, const Tensor& idx, const Tensor& dest_row, const optional<Tensor>& w,
                  int64_t H, int64_t E_local, std::vector<int64_t> flags, int64_t rank, int64_t world, int64_t epoch,
                  double limit_s, const optional<Tensor>& keep_rows, Tensor abort_word) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kInt && idx.dim() == 2 && idx.is_contiguous(), "ep_combine: idx i32 [T,k]");
  c10::cuda::CUDAGuard guard(idx.device());
  ferrl::EpCombineParams p{};
  p.ys = table_of_fwd(ys); p.idx = idx.data_ptr<int>(); p.dest_row = dest_row.data_ptr<int>();
  if (w.has_value() && w->defined()) {
    TORCH_CHECK(w->scalar_type() == at::kFloat && w->is_contiguous() && w->numel() == idx.numel(), "ep_combine: weights");
    p.w = w->data_ptr<float>();
  }
  p.T = idx.size(0); p.k = idx.size(1); p.H = H; p.E_local = E_local; p.rank = rank; p.world = world;
  p.flags = table_of_fwd(flags); p.epoch = static_cast<unsigned>(epoch);
  p.limit_ns = static_cast<unsigned long long>(limit_s * 1e9); p.status = status_word();
  p.abort_word = abort_word.data_ptr<int>();
  Tensor out = out_empty({p.T, H}, idx.options().dtype(at::kBFloat16));
  p.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  if (keep_rows.has_value() && keep_rows->defined()) {
    TORCH_CHECK(keep_rows->scalar_type() == at::kBFloat16 && keep_rows->is_contiguous() && keep_rows->numel() == idx.numel() * H, "ep_combine: keep_rows bf16 [T*k,H]");
    p.keep_rows = reinterpret_cast<__nv_bfloat16*>(keep_rows->data_ptr());
  }
  FERRL_CHECK(ferrl::ep_combine(p, num_sms(), stream()));
  return out;
}

// out[t] = sum_j w[t,j] * ys[row_of[t,j]]  (w undefined: plain sum)
Tensor moe_combine(const Tensor& ys, const Tensor& row_of, const optional<Tensor>& w, int64_t T, int64_t k) {
  TORCH_CHECK(ys.is_cuda() && ys.scalar_type() == at::kBFloat16 && ys.is_contiguous() && row_of.numel() == T * k, "moe_combine: shapes");
  c10::cuda::CUDAGuard guard(ys.device());
  Tensor out = out_empty({T, ys.size(1)}, ys.options());
  const float* wp = nullptr;
  if (w.has_value() && w->defined()) {
    TORCH_CHECK(w->scalar_type() == at::kFloat && w->is_contiguous() && w->numel() == T * k, "moe_combine: weights f32 [T,k]");
    wp = w->data_ptr<float>();
  }
  FERRL_CHECK(ferrl::moe_combine(ys.data_ptr(), row_of.data_ptr<int>(), wp, T, k, ys.size(1), out.data_ptr(), stream()));
  return out;
}

// dw[t,j] = <dy[t], ys[row_of[t,j]]>
Tensor moe_pair_dot(const Tensor& dy, const Tensor& ys, const Tensor& row_of, int64_t k) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kBFloat16 && dy.is_contiguous() && ys.is_contiguous() && dy.size(1) == ys.size(1), "moe_pair_dot: shapes");
  c10::cuda::CUDAGuard guard(dy.device());
  Tensor dw = out_empty({dy.size(0), k}, dy.options().dtype(at::kFloat));
  FERRL_CHECK(ferrl::moe_pair_dot(dy.data_ptr(), ys.data_ptr(), row_of.data_ptr<int>(), row_of.numel(), k, dy.size(1),
                                  dw.data_ptr<float>(), stream()));
  return dw;
}

std::tuple<Tensor, Tensor> rmsnorm(const Tensor& x, const optional<Tensor>& res, const optional<Tensor>& w,
                                   const optional<Tensor>& gate, double eps, bool zc) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "rmsnorm: contiguous CUDA tensor required");
  c10::cuda::CUDAGuard guard(x.device());
  const int H = x.size(-1);
  const long long rows = x.numel() / H;
  Tensor y = out_empty_like(x);
  Tensor h;
  if (res.has_value() && res->defined()) {
    TORCH_CHECK(res->is_contiguous() && res->sizes() == x.sizes() && res->scalar_type() == x.scalar_type(), "rmsnorm: residual");
    h = out_empty_like(x);
  }
  if (w.has_value() && w->defined()) TORCH_CHECK(w->scalar_type() == x.scalar_type() && w->numel() == H && w->is_contiguous(), "rmsnorm: weight");
  if (gate.has_value() && gate->defined()) TORCH_CHECK(gate->is_contiguous() && gate->sizes() == x.sizes() && gate->scalar_type() == x.scalar_type(), "rmsnorm: gate");
  FERRL_CHECK(ferrl::rmsnorm(dt(x), x.data_ptr(), optr(res), optr(w), optr(gate), y.data_ptr(),
                             h.defined() ? h.data_ptr() : nullptr, rows, H, static_cast<float>(eps), zc, stream()));
  return {y, h.defined() ? h : Tensor()};
}

Tensor rmsnorm_bwd(const Tensor& x, const optional<Tensor>& w, const Tensor& dy, double eps, bool zc) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && dy.is_contiguous() && dy.sizes() == x.sizes() &&
                  dy.scalar_type() == x.scalar_type(), "rmsnorm_bwd: shapes");
  c10::cuda::CUDAGuard guard(x.device());
  const int H = x.size(-1);
  Tensor dx = out_empty_like(x);
  FERRL_CHECK(ferrl::rmsnorm_bwd(dt(x), x.data_ptr(), optr(w), dy.data_ptr(), dx.data_ptr(), x.numel() / H, H,
                                 static_cast<float>(eps), zc, stream()));
  return dx;
}

std::tuple<Tensor, Tensor> rmsnorm_gated_bwd(const Tensor& x, const Tensor& gate, const Tensor& w, const Tensor& dy, double eps) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && gate.is_contiguous() && dy.is_contiguous() && w.is_contiguous() &&
                  dy.sizes() == x.sizes() && gate.sizes() == x.sizes() && dy.scalar_type() == x.scalar_type() &&
                  gate.scalar_type() == x.scalar_type() && w.scalar_type() == x.scalar_type() && w.numel() == x.size(-1),
              "rmsnorm_gated_bwd: x, gate, dy of one shape and dtype, w [H]");
  c10::cuda::CUDAGuard guard(x.device());
  const int H = x.size(-1);
  Tensor dx = out_empty_like(x), dg = out_empty_like(x);
  FERRL_CHECK(ferrl::rmsnorm_gated_bwd(dt(x), x.data_ptr(), gate.data_ptr(), w.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                       dg.data_ptr(), x.numel() / H, H, static_cast<float>(eps), stream()));
  return {dx, dg};
}

void fill_qknr(ferrl::QkNormRopeArgs& a, const Tensor& q, const Tensor& k, const optional<Tensor>& qw,
               const optional<Tensor>& kw, const Tensor& cos_t, const Tensor& sin_t, const Tensor& pos, int64_t pos_div,
               double eps, bool zc) {
  // q [T, Hq, D], k [T, Hkv, D]: heads packed (stride(1) == D, stride(2) == 1), arbitrary token stride
  TORCH_CHECK(q.is_cuda() && q.dim() == 3 && k.dim() == 3 && q.size(0) == k.size(0) && q.size(2) == k.size(2),
              "qk_norm_rope: q [T,Hq,D], k [T,Hkv,D]");
  TORCH_CHECK(q.stride(2) == 1 && k.stride(2) == 1 && q.stride(1) == q.size(2) && k.stride(1) == k.size(2),
              "qk_norm_rope: heads must be packed");
  TORCH_CHECK(q.scalar_type() == k.scalar_type(), "qk_norm_rope: dtype mismatch");
  TORCH_CHECK(cos_t.scalar_type() == at::kFloat && sin_t.scalar_type() == at::kFloat && cos_t.is_contiguous() &&
                  sin_t.is_contiguous() && cos_t.dim() == 2, "qk_norm_rope: float32 tables [max_pos, half]");
  TORCH_CHECK(pos.is_contiguous() && (pos.scalar_type() == at::kLong || pos.scalar_type() == at::kInt), "qk_norm_rope: positions int64/int32");
  a.dtype = dt(q);
  a.q_in = q.data_ptr(); a.ld_q = q.stride(0); a.k_in = k.data_ptr(); a.ld_k = k.stride(0);
  a.qw = optr(qw); a.kw = optr(kw);
  a.cos_t = cos_t.data_ptr<float>(); a.sin_t = sin_t.data_ptr<float>();
  a.pos64 = pos.scalar_type() == at::kLong ? reinterpret_cast<long long*>(pos.data_ptr<int64_t>()) : nullptr;
  a.pos32 = pos.scalar_type() == at::kInt ? pos.data_ptr<int>() : nullptr;
  a.pos_div = pos_div;
  a.n_tok = q.size(0); a.Hq = q.size(1); a.Hkv = k.size(1); a.D = q.size(2); a.half = cos_t.size(1);
  a.eps = static_cast<float>(eps); a.zero_centered = zc;
  TORCH_CHECK(pos.numel() * pos_div >= a.n_tok, "qk_norm_rope: too few positions");
}

std::tuple<Tensor, Tensor> qk_norm_rope_fwd(const Tensor& q, const Tensor& k, const optional<Tensor>& qw,
                                            const optional<Tensor>& kw, const Tensor& cos_t, const Tensor& sin_t,
                                            const Tensor& pos, int64_t pos_div, double eps, bool zc) {
  c10::cuda::CUDAGuard guard(q.device());
  ferrl::QkNormRopeArgs a{};
  fill_qknr(a, q, k, qw, kw, cos_t, sin_t, pos, pos_div, eps, zc);
  Tensor qo = out_empty({q.size(0), q.size(1), q.size(2)}, q.options());
  Tensor ko = out_empty({k.size(0), k.size(1), k.size(2)}, k.options());
  a.backward = false; a.q_out = qo.data_ptr(); a.k_out = ko.data_ptr();
  FERRL_CHECK(ferrl::qk_norm_rope(a, stream()));
  return {qo, ko};
}

// Decode form: one token per row; the rotated keys and the values go straight into the KV cache
// (dense [B, Smax, Hkv, D], or a paged pool [n_pages, page, Hkv, D] behind `table`), only q is returned.
Tensor qk_norm_rope_append(const Tensor& q, const Tensor& k, const Tensor& v, const optional<Tensor>& qw,
                           const optional<Tensor>& kw, const Tensor& cos_t, const Tensor& sin_t, const Tensor& pos,
                           double eps, bool zc, Tensor kc, Tensor vc, const Tensor& kv_len, const optional<Tensor>& table) {
  c10::cuda::CUDAGuard guard(q.device());
  ferrl::QkNormRopeArgs a{};
  fill_qknr(a, q, k, qw, kw, cos_t, sin_t, pos, 1, eps, zc);
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16 && v.dim() == 3 && v.sizes() == k.sizes() &&
                  v.stride(2) == 1 && v.stride(1) == v.size(2) && kc.is_contiguous() && vc.is_contiguous() &&
                  kc.dim() == 4 && kc.sizes() == vc.sizes() && kc.size(2) == k.size(1) && kc.size(3) == k.size(2) &&
                  kv_len.scalar_type() == at::kInt && kv_len.is_contiguous() && kv_len.numel() == q.size(0),
              "qk_norm_rope_append: layout");
  Tensor qo = out_empty({q.size(0), q.size(1), q.size(2)}, q.options());
  a.backward = false; a.q_out = qo.data_ptr(); a.k_out = nullptr;
  a.kc = kc.data_ptr(); a.vc = vc.data_ptr(); a.v_in = v.data_ptr(); a.ld_v = v.stride(0);
  a.kv_len = kv_len.data_ptr<int>();
  if (table.has_value() && table->defined()) {
    TORCH_CHECK(table->scalar_type() == at::kInt && table->dim() == 2 && table->stride(1) == 1 && table->size(0) == q.size(0),
                "qk_norm_rope_append: table int32 [B, pages]");
    a.table = table->data_ptr<int>(); a.bt_stride = table->stride(0); a.page = kc.size(1);
  } else {
    TORCH_CHECK(kc.size(0) == q.size(0), "qk_norm_rope_append: dense cache [B, Smax, Hkv, D]");
    a.smax = kc.size(1);
  }
  FERRL_CHECK(ferrl::qk_norm_rope(a, stream()));
  return qo;
}

// d(q_in), d(k_in) written into dq_in / dk_in (views with packed heads, any token stride)
void qk_norm_rope_bwd(const Tensor& q, const Tensor& k, const optional<Tensor>& qw, const optional<Tensor>& kw,
                      const Tensor& cos_t, const Tensor& sin_t, const Tensor& pos, int64_t pos_div, double eps, bool zc,
                      const Tensor& dq, const Tensor& dk, Tensor dq_in, Tensor dk_in) {
  c10::cuda::CUDAGuard guard(q.device());
  ferrl::QkNormRopeArgs a{};
  fill_qknr(a, q, k, qw, kw, cos_t, sin_t, pos, pos_div, eps, zc);
  TORCH_CHECK(dq.is_contiguous() && dk.is_contiguous() && dq_in.sizes() == q.sizes() && dk_in.sizes() == k.sizes() &&
                  dq_in.stride(2) == 1 && dk_in.stride(2) == 1 && dq_in.stride(1) == q.size(2) &&
                  dk_in.stride(1) == k.size(2), "qk_norm_rope_bwd: shapes");
  a.backward = true; a.dq = dq.data_ptr(); a.dk = dk.data_ptr();
  a.q_out = dq_in.data_ptr(); a.k_out = dk_in.data_ptr(); a.ld_dq = dq_in.stride(0); a.ld_dk = dk_in.stride(0);
  FERRL_CHECK(ferrl::qk_norm_rope(a, stream()));
}

void kv_append(const Tensor& k, const Tensor& v, Tensor kc, Tensor vc, const Tensor& kv_len) {
  // k [B, Hkv*D] contiguous, v [B, Hkv*D] row-strided view, caches [B, Smax, Hkv, D]
  c10::cuda::CUDAGuard guard(k.device());
  TORCH_CHECK(k.is_contiguous() && v.stride(-1) == 1 && kc.is_contiguous() && vc.is_contiguous() &&
                  kv_len.scalar_type() == at::kInt, "kv_append: layout");
  const int B = kc.size(0), smax = kc.size(1), HD = kc.size(2) * kc.size(3);
  FERRL_CHECK(ferrl::kv_append(dt(k), k.data_ptr(), v.data_ptr(), v.stride(0), kc.data_ptr(), vc.data_ptr(),
                               kv_len.data_ptr<int>(), B, smax, HD, stream()));
}

void kv_append_paged(const Tensor& k, const Tensor& v, Tensor kc, Tensor vc, const Tensor& kv_len, const Tensor& table) {
  // k [B, Hkv*D] contiguous, v [B, Hkv*D] row-strided view, pools [n_pages, page, Hkv, D], table [B, max_pages] i32
  c10::cuda::CUDAGuard guard(k.device());
  TORCH_CHECK(k.scalar_type() == at::kBFloat16 && k.is_contiguous() && v.stride(-1) == 1 && kc.is_contiguous() &&
                  vc.is_contiguous() && kc.dim() == 4 && kv_len.scalar_type() == at::kInt && table.scalar_type() == at::kInt &&
                  table.dim() == 2 && table.is_contiguous() && table.size(0) == k.size(0), "kv_append_paged: layout");
  FERRL_CHECK(ferrl::kv_append_paged(k.data_ptr(), v.data_ptr(), v.stride(0), kc.data_ptr(), vc.data_ptr(),
                                     kv_len.data_ptr<int>(), table.data_ptr<int>(), table.size(1), kc.size(1), k.size(0),
                                     kc.size(2) * kc.size(3), stream()));
}

Tensor glu_fwd(const Tensor& gu, int64_t act) {
  TORCH_CHECK(gu.is_cuda() && gu.is_contiguous(), "glu: contiguous CUDA tensor");
  c10::cuda::CUDAGuard guard(gu.device());
  const int F = gu.size(-1) / 2;
  auto sizes = gu.sizes().vec();
  sizes.back() = F;
  Tensor out = out_empty(sizes, gu.options());
  FERRL_CHECK(ferrl::glu(dt(gu), false, gu.data_ptr(), nullptr, out.data_ptr(), gu.numel() / (2 * F), F, act, stream()));
  return out;
}

Tensor glu_bwd(const Tensor& gu, const Tensor& dout, int64_t act) {
  TORCH_CHECK(gu.is_contiguous() && dout.is_contiguous(), "glu_bwd: contiguous");
  c10::cuda::CUDAGuard guard(gu.device());
  const int F = gu.size(-1) / 2;
  Tensor dgu = out_empty_like(gu);
  FERRL_CHECK(ferrl::glu(dt(gu), true, gu.data_ptr(), dout.data_ptr(), dgu.data_ptr(), gu.numel() / (2 * F), F, act, stream()));
  return dgu;
}

Tensor embedding(const Tensor& ids, const Tensor& table, double scale) {
  TORCH_CHECK(ids.scalar_type() == at::kLong && table.is_contiguous() && table.dim() == 2, "embedding: args");
  c10::cuda::CUDAGuard guard(table.device());
  Tensor idc = ids.contiguous();
  auto sizes = idc.sizes().vec();
  sizes.push_back(table.size(1));
  Tensor out = out_empty(sizes, table.options());
  FERRL_CHECK(ferrl::embedding(dt(table), reinterpret_cast<long long*>(idc.data_ptr<int64_t>()), table.data_ptr(), out.data_ptr(), idc.numel(),
                               table.size(1), table.size(0), static_cast<float>(scale), stream()));
  return out;
}

Tensor lora_merge(const Tensor& w, const Tensor& a, const Tensor& b) {
  TORCH_CHECK(w.is_contiguous() && a.is_contiguous() && b.is_contiguous() && a.scalar_type() == at::kFloat &&
                  b.scalar_type() == at::kFloat && a.size(1) == w.size(1) && b.size(0) == w.size(0) &&
                  a.size(0) == b.size(1), "lora_merge: shapes");
  c10::cuda::CUDAGuard guard(w.device());
  Tensor out = out_empty_like(w);
  FERRL_CHECK(ferrl::lora_merge(dt(w), w.data_ptr(), a.data_ptr<float>(), b.data_ptr<float>(), out.data_ptr(),
                                w.size(0), w.size(1), a.size(0), stream()));
  return out;
}

// Multi-tensor AdamW with optional in-kernel global-norm clip. Returns the pre-clip gradient norm
// (a 1-element device tensor; zeros when compute_norm is false).
Tensor adamw_step(std::vector<Tensor> params, std::vector<Tensor> grads, std::vector<Tensor> m, std::vector<Tensor> v,
                  double lr, double b1, double b2, double eps, double wd, int64_t step, double max_norm,
                  double pre_scale, bool compute_norm) {
  const size_t n = params.size();
  TORCH_CHECK(grads.size() == n && m.size() == n && v.size() == n, "adamw: list sizes");
  Tensor norm = out_zeros({1}, at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, c10::cuda::current_device()));
  if (n == 0) return norm;
  c10::cuda::CUDAGuard guard(params[0].device());
  const int chunk = 1 << 16;
  std::vector<ferrl::AdamTensor> tab(n);
  std::vector<int> blk_t;
  std::vector<long long> blk_o;
  for (size_t i = 0; i < n; ++i) {
    TORCH_CHECK(params[i].scalar_type() == at::kFloat && grads[i].scalar_type() == at::kFloat &&
                    params[i].is_contiguous() && grads[i].is_contiguous() && m[i].is_contiguous() &&
                    v[i].is_contiguous() && grads[i].numel() == params[i].numel(), "adamw: float32 contiguous tensors");
    tab[i] = {params[i].data_ptr<float>(), grads[i].data_ptr<float>(), m[i].data_ptr<float>(), v[i].data_ptr<float>(),
              params[i].numel()};
    for (long long o = 0; o < params[i].numel(); o += chunk) {
      blk_t.push_back(static_cast<int>(i));
      blk_o.push_back(o);
    }
  }
  const size_t tab_b = n * sizeof(ferrl::AdamTensor), bt_b = blk_t.size() * sizeof(int), bo_b = blk_o.size() * sizeof(long long);
  const size_t off1 = (tab_b + 15) & ~size_t(15), off2 = (off1 + bt_b + 15) & ~size_t(15), total = off2 + bo_b + 16;
  Tensor host = out_empty({static_cast<long long>(total)}, at::TensorOptions().dtype(at::kByte).pinned_memory(true));
  memcpy(host.data_ptr<uint8_t>(), tab.data(), tab_b);
  memcpy(host.data_ptr<uint8_t>() + off1, blk_t.data(), bt_b);
  memcpy(host.data_ptr<uint8_t>() + off2, blk_o.data(), bo_b);
  Tensor dev = host.to(params[0].device(), /*non_blocking=*/true);
  Tensor sumsq = out_zeros({1}, norm.options().dtype(at::kDouble));
  uint8_t* d = dev.data_ptr<uint8_t>();
  const float bc1 = 1.f / (1.f - static_cast<float>(std::pow(b1, static_cast<double>(step))));
  const float bc2 = 1.f / (1.f - static_cast<float>(std::pow(b2, static_cast<double>(step))));
  FERRL_CHECK(ferrl::adamw_multi(reinterpret_cast<ferrl::AdamTensor*>(d), reinterpret_cast<int*>(d + off1),
                                 reinterpret_cast<long long*>(d + off2), static_cast<int>(blk_t.size()), chunk,
                                 sumsq.data_ptr<double>(), compute_norm, lr, b1, b2, eps, wd, bc1, bc2,
                                 static_cast<float>(max_norm), static_cast<float>(pre_scale), norm.data_ptr<float>(),
                                 stream()));
  return norm;
}

std::tuple<Tensor, Tensor, Tensor> grpo_loss_rows(const Tensor& logp, const Tensor& logp_old,
                                                  const optional<Tensor>& logp_ref, const Tensor& adv,
                                                  const Tensor& mask, const optional<Tensor>& tis, double eps_lo,
                                                  double eps_hi, double beta, bool seq_level, bool want_grad) {
  TORCH_CHECK(logp.is_cuda() && logp.scalar_type() == at::kFloat && logp.is_contiguous() && logp_old.is_contiguous() &&
                  mask.is_contiguous() && adv.is_contiguous() && logp.dim() == 2, "grpo_loss: float32 [G,L] tensors");
  c10::cuda::CUDAGuard guard(logp.device());
  const int G = logp.size(0), L = logp.size(1);
  Tensor row_sum = out_empty({G}, logp.options()), row_cnt = out_empty({G}, logp.options());
  Tensor dl = want_grad ? out_empty_like(logp) : Tensor();
  int mode = (seq_level ? 1 : 0) | (logp_ref.has_value() && logp_ref->defined() ? 2 : 0) |
             (tis.has_value() && tis->defined() ? 4 : 0);
  FERRL_CHECK(ferrl::grpo_loss_rows(logp.data_ptr<float>(), logp_old.data_ptr<float>(),
                                    static_cast<const float*>(optr(logp_ref)), adv.data_ptr<float>(),
                                    mask.data_ptr<float>(), static_cast<const float*>(optr(tis)),
                                    row_sum.data_ptr<float>(), row_cnt.data_ptr<float>(),
                                    want_grad ? dl.data_ptr<float>() : nullptr, G, L, eps_lo, eps_hi, beta, mode, stream()));
  return {row_sum, row_cnt, dl};
}

void grpo_scale_rows(Tensor dlogp, const Tensor& row_scale) {
  c10::cuda::CUDAGuard guard(dlogp.device());
  FERRL_CHECK(ferrl::grpo_scale_rows(dlogp.data_ptr<float>(), row_scale.data_ptr<float>(), dlogp.size(0), dlogp.size(1), stream()));
}

Tensor decode_attn(const Tensor& q, const Tensor& kc, const Tensor& vc, const Tensor& kv_len, double scale,
                   int64_t window, int64_t n_splits, const optional<Tensor>& block_table, int64_t page, int64_t variant,
                   const optional<Tensor>& prefix_len, int64_t group, int64_t prefix_splits) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.is_contiguous() && q.dim() == 3, "decode_attn: q bf16 [B,Hq,D]");
  TORCH_CHECK(kc.scalar_type() == at::kBFloat16 && kc.is_contiguous() && vc.is_contiguous() && kc.dim() == 4, "decode_attn: caches bf16 [B,S,Hkv,D]");
  TORCH_CHECK(kv_len.scalar_type() == at::kInt && kv_len.is_contiguous(), "decode_attn: kv_len int32");
  c10::cuda::CUDAGuard guard(q.device());
  ferrl::DecodeAttnArgs a{};
  a.B = q.size(0); a.Hq = q.size(1); a.D = q.size(2); a.Hkv = kc.size(2);
  a.q = q.data_ptr(); a.k = kc.data_ptr(); a.v = vc.data_ptr(); a.kv_len = kv_len.data_ptr<int>();
  a.seq_stride = kc.stride(0); a.tok_stride = kc.stride(1);
  if (block_table.has_value() && block_table->defined()) {
    TORCH_CHECK(block_table->scalar_type() == at::kInt && block_table->is_contiguous(), "decode_attn: block_table int32");
    a.block_table = block_table->data_ptr<int>(); a.bt_stride = block_table->size(1); a.page = page;
  }
  a.scale = scale; a.window = window;
  a.n_splits = n_splits > 0 ? n_splits : ferrl::decode_attn_pick_splits(a.B, a.Hkv, kc.size(1), num_sms());
  Tensor out = out_empty_like(q);
  Tensor ws;
  if (prefix_len.has_value() && prefix_len->defined()) {
    TORCH_CHECK(prefix_len->scalar_type() == at::kInt && prefix_len->is_contiguous() && group >= 1 &&
                    prefix_len->numel() * group == a.B, "decode_attn: prefix_len int32 [B / group]");
    a.prefix_len = prefix_len->data_ptr<int>(); a.group = static_cast<int>(group);
    a.prefix_splits = static_cast<int>(prefix_splits);
    a.n_splits = 1;
    ws = out_empty({static_cast<long long>(a.B) * a.Hq * a.prefix_splits * (a.D + 2)}, q.options().dtype(at::kFloat));
    a.workspace = ws.data_ptr<float>();
  } else if (a.n_splits > 1) {
    ws = out_empty({static_cast<long long>(ferrl::decode_attn_workspace_bytes(a.B, a.Hq, a.D, a.n_splits) / 4)},
                   q.options().dtype(at::kFloat));
    a.workspace = ws.data_ptr<float>();
  }
  a.out = out.data_ptr();
  a.no_pipe = static_cast<int>(variant);
  FERRL_CHECK(ferrl::decode_attn(a, stream()));
  return out;
}

void fill_flash(ferrl::FlashArgs& a, const Tensor& q, const Tensor& k, const Tensor& v, double scale, bool causal,
                int64_t window, int64_t q_offset) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
                  v.scalar_type() == at::kBFloat16, "flash: bf16 tensors");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "flash: [B,S,H,D] tensors");
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1 && q.stride(2) == q.size(3) &&
                  k.stride(2) == k.size(3) && v.stride(2) == v.size(3), "flash: heads must be packed along the last dims");
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr();
  a.q_bs = q.stride(0); a.q_ts = q.stride(1); a.k_bs = k.stride(0); a.k_ts = k.stride(1);
  a.v_bs = v.stride(0); a.v_ts = v.stride(1);
  a.B = q.size(0); a.Sq = q.size(1); a.Sk = k.size(1); a.Hq = q.size(2); a.Hkv = k.size(2); a.D = q.size(3);
  a.scale = scale; a.causal = causal; a.window = window; a.q_offset = q_offset;
}

// variant: 0 = tcgen05 kernel where it applies (causal self-attention, head_dim 128), 1 = warp-level kernel,
// 2 = tcgen05 kernel with the output kept in TMEM and rescaled lazily
std::tuple<Tensor, Tensor> flash_fwd(const Tensor& q, const Tensor& k, const Tensor& v, double scale, bool causal,
                                     int64_t window, int64_t q_offset, int64_t variant) {
  c10::cuda::CUDAGuard guard(q.device());
  ferrl::FlashArgs a{};
  fill_flash(a, q, k, v, scale, causal, window, q_offset);
  Tensor o = out_empty({a.B, a.Sq, a.Hq, a.D}, q.options());
  Tensor lse = out_empty({a.B, a.Hq, a.Sq}, q.options().dtype(at::kFloat));
  a.o = o.data_ptr(); a.o_bs = o.stride(0); a.o_ts = o.stride(1); a.lse = lse.data_ptr<float>();
  if ((variant == 0 || variant == 2 || variant == 3) && ferrl::flash_fwd_tc_supported(a)) {
    Tensor vt = out_empty({static_cast<long long>(ferrl::flash_fwd_tc_workspace_elems(a))}, q.options());
    // variant 0: output and P in TMEM (default); 3: output in TMEM, P through shared memory; 2: first form (output in registers)
    FERRL_CHECK(ferrl::flash_fwd_tc(a, vt.data_ptr(), status_word(), stream(), variant == 0 ? 2 : (variant == 3 ? 1 : 0)));
    return {o, lse};
  }
  FERRL_CHECK(ferrl::flash_fwd(a, stream()));
  return {o, lse};
}

std::tuple<Tensor, Tensor, Tensor> flash_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                             const Tensor& lse, const Tensor& d_o, double scale, bool causal,
                                             int64_t window, int64_t q_offset, int64_t variant,
                                             const optional<Tensor>& debug) {
  c10::cuda::CUDAGuard guard(q.device());
  ferrl::FlashArgs a{};
  fill_flash(a, q, k, v, scale, causal, window, q_offset);
  TORCH_CHECK(o.is_contiguous() && d_o.is_contiguous() && lse.is_contiguous(), "flash_bwd: o, do, lse contiguous");
  Tensor dq = out_empty({a.B, a.Sq, a.Hq, a.D}, q.options());
  Tensor dk = out_empty({a.B, a.Sk, a.Hkv, a.D}, q.options());
  Tensor dv = out_empty({a.B, a.Sk, a.Hkv, a.D}, q.options());
  Tensor delta = out_empty({a.B, a.Hq, a.Sq}, lse.options());
  a.o = o.data_ptr(); a.o_bs = o.stride(0); a.o_ts = o.stride(1); a.lse = lse.data_ptr<float>();
  a.d_o = d_o.data_ptr(); a.do_bs = d_o.stride(0); a.do_ts = d_o.stride(1);
  a.dq = dq.data_ptr(); a.dq_bs = dq.stride(0); a.dq_ts = dq.stride(1);
  a.dk = dk.data_ptr(); a.dk_bs = dk.stride(0); a.dk_ts = dk.stride(1);
  a.dv = dv.data_ptr(); a.dv_bs = dv.stride(0); a.dv_ts = dv.stride(1);
  a.delta = delta.data_ptr<float>();
  if (debug.has_value() && debug->defined()) {
    TORCH_CHECK(debug->scalar_type() == at::kLong && debug->is_contiguous() && debug->numel() >= 1024, "flash_bwd: debug int64[>=1024]");
    a.debug = reinterpret_cast<unsigned long long*>(debug->data_ptr<int64_t>());
  }
  // variant 0: tcgen05 kernels where they apply; 1: warp-level kernels
  if (variant != 1 && ferrl::flash_bwd_tc_supported(a)) {
    Tensor stats = out_empty({static_cast<long long>(ferrl::flash_bwd_tc_scratch_floats(a))}, lse.options());
    a.delta = stats.data_ptr<float>();
    FERRL_CHECK(ferrl::flash_bwd_tc(a, status_word(), stream()));
    return {dq, dk, dv};
  }
  FERRL_CHECK(ferrl::flash_bwd(a, stream()));
  return {dq, dk, dv};
}

static void lp_head_common(ferrl::GemmArgs& a, const Tensor& hidden, const Tensor& w, const Tensor& targets, double temperature,
                           double softcap, const char* what) {
  TORCH_CHECK(hidden.is_cuda() && hidden.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && hidden.dim() == 2 &&
                  w.dim() == 2 && hidden.size(1) == w.size(1) && hidden.stride(1) == 1 && w.stride(1) == 1,
              what, ": hidden [M,H] and weight [V,H] bf16, K-major");
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == hidden.size(0), what, ": targets int64 [M]");
  a.A = hidden.data_ptr(); a.B = w.data_ptr(); a.lda = hidden.stride(0); a.ldb = w.stride(0);
  a.M = hidden.size(0); a.N = w.size(0); a.K = hidden.size(1);
  a.status = status_word(); a.num_sms = num_sms();
  a.lp_targets = reinterpret_cast<const long long*>(targets.data_ptr<int64_t>());
  a.lp_inv_t = static_cast<float>(1.0 / temperature);
  a.lp_cap = static_cast<float>(softcap);
  // the two-SM kernel for training-sized row counts, the one-SM kernel (256-wide tiles) below that
  if (a.M >= 1024 && a.N >= 512) a.two_cta = 256; else a.force_bn = 256;
}

// log_softmax(softcap(h W^T) / T)[target] per row with the row statistics taken in the head GEMM's epilogue:
// no [M, V] tensor exists at any point.  Returns (lp [M], lse [M]) in fp32.
std::tuple<Tensor, Tensor> logprob_head_fwd(const Tensor& hidden, const Tensor& w, const Tensor& targets, double temperature,
                                            double softcap) {
  ferrl::GemmArgs a{};
  lp_head_common(a, hidden, w, targets, temperature, softcap, "logprob_head_fwd");
  c10::cuda::CUDAGuard guard(hidden.device());
  const int n_tiles = (a.N + 255) / 256;
  auto f32 = hidden.options().dtype(at::kFloat);
  Tensor ws = out_empty({n_tiles, a.M, 2}, f32), tl = out_zeros({a.M}, f32);
  Tensor lp = out_empty({a.M}, f32), lse = out_empty({a.M}, f32);
  if (a.M == 0) return {lp, lse};
  a.lp_mode = 1; a.lp_ws = ws.data_ptr<float>(); a.lp_tl = tl.data_ptr<float>(); a.ldo = a.N;
  FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
  FERRL_CHECK(ferrl::logprob_finalize(ws.data_ptr<float>(), tl.data_ptr<float>(), n_tiles, a.M, lp.data_ptr<float>(),
                                      lse.data_ptr<float>(), stream()));
  return {lp, lse};
}

// One vocabulary shard of the head (rows col0 .. col0 + Vs of the full head): per row (max, sum exp(z - max), target
// logit or 0 when the target lies in another shard), fp32 [M, 3].  The caller merges the shards' partials.
Tensor logprob_head_shard_stats(const Tensor& hidden, const Tensor& w, const Tensor& targets, double temperature, double softcap,
                                int64_t col0) {
  ferrl::GemmArgs a{};
  lp_head_common(a, hidden, w, targets, temperature, softcap, "logprob_head_shard_stats");
  c10::cuda::CUDAGuard guard(hidden.device());
  const int n_tiles = (a.N + 255) / 256;
  auto f32 = hidden.options().dtype(at::kFloat);
  Tensor ws = out_empty({n_tiles, a.M, 2}, f32), tl = out_zeros({a.M}, f32), stats = out_empty({a.M, 3}, f32);
  if (a.M == 0) return stats;
  a.lp_mode = 1; a.lp_ws = ws.data_ptr<float>(); a.lp_tl = tl.data_ptr<float>(); a.ldo = a.N; a.lp_col0 = col0;
  FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
  FERRL_CHECK(ferrl::logprob_shard_stats(ws.data_ptr<float>(), tl.data_ptr<float>(), n_tiles, a.M, stats.data_ptr<float>(), stream()));
  return stats;
}

// Gradient of sum_rows coef[row] * (-lp[row]) with respect to the raw logits of the vocabulary slice `w`
// ([Vc, H] rows col0 .. col0+Vc of the head), written as bf16 [M, Vc]: the softmax is recomputed in the
// GEMM epilogue from the saved lse.
Tensor logprob_head_dlogits(const Tensor& hidden, const Tensor& w, const Tensor& targets, const Tensor& lse, const Tensor& coef,
                            double temperature, double softcap, int64_t col0) {
  ferrl::GemmArgs a{};
  lp_head_common(a, hidden, w, targets, temperature, softcap, "logprob_head_dlogits");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && coef.scalar_type() == at::kFloat && lse.is_contiguous() && coef.is_contiguous() &&
                  lse.numel() == a.M && coef.numel() == a.M, "logprob_head_dlogits: lse, coef fp32 [M]");
  c10::cuda::CUDAGuard guard(hidden.device());
  Tensor out = out_empty({a.M, a.N}, hidden.options());
  if (a.M == 0) return out;
  a.lp_mode = 2; a.lp_lse = lse.data_ptr<float>(); a.lp_coef = coef.data_ptr<float>(); a.lp_col0 = col0;
  a.out = out.data_ptr(); a.ldo = a.N;
  FERRL_CHECK(ferrl::gemm_bf16(a, stream()));
  return out;
}

std::tuple<Tensor, Tensor> logprob_rows(const Tensor& logits, const Tensor& targets, double temperature, double softcap) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1 && targets.scalar_type() == at::kLong &&
                  targets.is_contiguous() && targets.numel() == logits.size(0), "logprob_rows: args");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor lp = out_empty({logits.size(0)}, logits.options().dtype(at::kFloat)), lse = out_empty_like(lp);
  FERRL_CHECK(ferrl::logprob_rows(dt(logits), logits.data_ptr(), logits.stride(0), reinterpret_cast<long long*>(targets.data_ptr<int64_t>()),
                                  lp.data_ptr<float>(), lse.data_ptr<float>(), logits.size(0), logits.size(1),
                                  temperature, softcap, stream()));
  return {lp, lse};
}

void logprob_rows_bwd(Tensor logits, const Tensor& targets, const Tensor& lse, const Tensor& dlp, double temperature,
                      double softcap) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(dlp.scalar_type() == at::kFloat && dlp.is_contiguous() && lse.is_contiguous(), "logprob_rows_bwd: args");
  FERRL_CHECK(ferrl::logprob_rows_bwd(dt(logits), logits.data_ptr(), logits.stride(0), reinterpret_cast<long long*>(targets.data_ptr<int64_t>()),
                                      lse.data_ptr<float>(), dlp.data_ptr<float>(), logits.size(0), logits.size(1),
                                      temperature, softcap, stream()));
}

std::tuple<Tensor, Tensor> sample_rows(const Tensor& logits, const Tensor& global_rows, int64_t seed,
                                       const optional<Tensor>& draw_dev, int64_t draw, double temperature, double top_p) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1 && global_rows.scalar_type() == at::kLong &&
                  global_rows.is_contiguous() && global_rows.numel() == logits.size(0), "sample_rows: args");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor tok = out_empty({logits.size(0)}, logits.options().dtype(at::kLong));
  Tensor lp = out_empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  const int* dd = nullptr;
  if (draw_dev.has_value() && draw_dev->defined()) {
    TORCH_CHECK(draw_dev->scalar_type() == at::kInt, "sample_rows: draw counter int32");
    dd = draw_dev->data_ptr<int>();
  }
  FERRL_CHECK(ferrl::sample_rows(dt(logits), logits.data_ptr(), logits.stride(0), reinterpret_cast<long long*>(global_rows.data_ptr<int64_t>()),
                                 static_cast<unsigned long long>(seed), dd, draw, reinterpret_cast<long long*>(tok.data_ptr<int64_t>()),
                                 lp.data_ptr<float>(), logits.size(0), logits.size(1), temperature, top_p, stream()));
  return {tok, lp};
}

// ------------------------------------------------------------------ symmetric heap
Tensor symm_alloc(int64_t nbytes) {
  void* ptr = nullptr;
  C10_CUDA_CHECK(cudaMalloc(&ptr, nbytes));
  C10_CUDA_CHECK(cudaMemset(ptr, 0, nbytes));
  int dev = c10::cuda::current_device();
  return at::from_blob(ptr, {nbytes}, [](void* p) { cudaFree(p); },
                       at::TensorOptions().dtype(at::kByte).device(at::kCUDA, dev));
}

Tensor symm_handle(const Tensor& buf) {
  cudaIpcMemHandle_t h;
  C10_CUDA_CHECK(cudaIpcGetMemHandle(&h, buf.data_ptr()));
  Tensor out = out_empty({static_cast<long long>(sizeof(h))}, at::TensorOptions().dtype(at::kByte));
  memcpy(out.data_ptr(), &h, sizeof(h));
  return out;
}

int64_t symm_open(const Tensor& handle) {
  TORCH_CHECK(!handle.is_cuda() && handle.numel() == static_cast<long long>(sizeof(cudaIpcMemHandle_t)), "symm_open: handle bytes");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle.data_ptr(), sizeof(h));
  void* ptr = nullptr;
  C10_CUDA_CHECK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return reinterpret_cast<int64_t>(ptr);
}

void symm_close(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }

ferrl::PeerTable table_of(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() <= ferrl::kMaxRanks, "too many ranks");
  ferrl::PeerTable t{};
  for (size_t i = 0; i < ptrs.size(); ++i) t.ptr[i] = reinterpret_cast<void*>(ptrs[i]);
  return t;
}

// Fused DP step; `tables` is a device uint8 blob holding [AdamTensor x n | blk_tensor | blk_off | blk_flat]
// laid out by the caller (offsets in bytes), `out` a float32[3] device tensor.
void dp_step(std::vector<int64_t> grads, std::vector<int64_t> reduced, std::vector<int64_t> flags,
             std::vector<int64_t> scalars, int64_t rank, int64_t world, int64_t barrier_world, int64_t own_lo,
             int64_t own_hi, int64_t n, int64_t epoch, double pre_scale, double uncovered_local, const Tensor& tables,
             int64_t off_blk_tensor, int64_t off_blk_off, int64_t off_blk_flat, int64_t n_blocks, int64_t chunk,
             double lr, double b1, double b2, double eps, double wd, int64_t step, double max_norm,
             Tensor block_partials, Tensor out, Tensor abort_word, double limit_s) {
  c10::cuda::CUDAGuard guard(out.device());
  ferrl::DpStepParams p{};
  p.grads = table_of(grads); p.reduced = table_of(reduced); p.flags = table_of(flags); p.scalars = table_of(scalars);
  p.rank = rank; p.world = world; p.barrier_world = barrier_world; p.own_lo = own_lo; p.own_hi = own_hi;
  p.n = n; p.epoch = static_cast<unsigned>(epoch); p.pre_scale = pre_scale; p.uncovered_local = uncovered_local;
  uint8_t* d = tables.data_ptr<uint8_t>();
  p.tab = reinterpret_cast<const ferrl::AdamTensor*>(d);
  p.blk_tensor = reinterpret_cast<const int*>(d + off_blk_tensor);
  p.blk_off = reinterpret_cast<const long long*>(d + off_blk_off);
  p.blk_flat = reinterpret_cast<const long long*>(d + off_blk_flat);
  p.n_blocks = n_blocks; p.chunk = chunk;
  p.lr = lr; p.b1 = b1; p.b2 = b2; p.eps = eps; p.wd = wd;
  p.bc1_inv = 1.f / (1.f - static_cast<float>(std::pow(b1, static_cast<double>(step))));
  p.bc2_inv = 1.f / (1.f - static_cast<float>(std::pow(b2, static_cast<double>(step))));
  p.max_norm = max_norm;
  TORCH_CHECK(block_partials.scalar_type() == at::kDouble && block_partials.numel() >= 2 * ferrl::dp_step_grid(num_sms()), "dp_step: block_partials too small");
  p.block_partials = block_partials.data_ptr<double>();
  p.out = out.data_ptr<float>(); p.status = status_word(); p.abort_word = abort_word.data_ptr<int>();
  p.limit_ns = static_cast<unsigned long long>(limit_s * 1e9);
  FERRL_CHECK(ferrl::dp_step(p, num_sms(), stream()));
}

// Packs the AdamW tensor table for dp_step / reuse; returns (device blob, off_blk_tensor, off_blk_off, off_blk_flat, n_blocks)
std::tuple<Tensor, int64_t, int64_t, int64_t, int64_t> dp_tables(std::vector<Tensor> params, std::vector<Tensor> m,
                                                                std::vector<Tensor> v, std::vector<int64_t> flat_off,
                                                                int64_t chunk) {
  const size_t n = params.size();
  std::vector<ferrl::AdamTensor> tab(n);
  std::vector<int> bt; std::vector<long long> bo, bf;
  for (size_t i = 0; i < n; ++i) {
    TORCH_CHECK(params[i].scalar_type() == at::kFloat && params[i].is_contiguous() && m[i].is_contiguous() && v[i].is_contiguous(), "dp_tables: float32 contiguous");
    tab[i] = {params[i].data_ptr<float>(), nullptr, m[i].data_ptr<float>(), v[i].data_ptr<float>(), params[i].numel()};
    for (long long o = 0; o < params[i].numel(); o += chunk) { bt.push_back(i); bo.push_back(o); bf.push_back(flat_off[i] + o); }
  }
  auto al = [](size_t x) { return (x + 15) & ~size_t(15); };
  size_t o1 = al(n * sizeof(ferrl::AdamTensor)), o2 = al(o1 + bt.size() * 4), o3 = al(o2 + bo.size() * 8), tot = o3 + bf.size() * 8 + 16;
  Tensor host = out_empty({static_cast<long long>(tot)}, at::TensorOptions().dtype(at::kByte));
  uint8_t* h = host.data_ptr<uint8_t>();
  memcpy(h, tab.data(), n * sizeof(ferrl::AdamTensor));
  memcpy(h + o1, bt.data(), bt.size() * 4);
  memcpy(h + o2, bo.data(), bo.size() * 8);
  memcpy(h + o3, bf.data(), bf.size() * 8);
  return {host.to(params[0].device()), static_cast<int64_t>(o1), static_cast<int64_t>(o2), static_cast<int64_t>(o3), static_cast<int64_t>(bt.size())};
}

void symm_all_reduce(std::vector<int64_t> src, std::vector<int64_t> flags, Tensor out, int64_t rank, int64_t world,
                     int64_t epoch, double limit_s, Tensor abort_word) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_contiguous(), "symm_all_reduce: contiguous output");
  FERRL_CHECK(ferrl::symm_all_reduce(dt(out), table_of(src), table_of(flags), out.data_ptr(), out.numel(), rank, world,
                                     static_cast<unsigned>(epoch), static_cast<unsigned long long>(limit_s * 1e9),
                                     status_word(), abort_word.data_ptr<int>(), num_sms(), stream()));
}

void symm_row_collective(int64_t which, std::vector<int64_t> src, std::vector<int64_t> flags, Tensor out, int64_t n_shard, int64_t rank,
                         int64_t world, int64_t epoch, double limit_s, Tensor abort_word) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_contiguous() && (which == 0 ? out.numel() == n_shard : out.numel() == n_shard * world),
              "symm_row_collective: contiguous output of n_shard (reduce-scatter) or world * n_shard (all-gather) elements");
  FERRL_CHECK(ferrl::symm_row_collective(static_cast<int>(which), dt(out), table_of(src), table_of(flags), out.data_ptr(), n_shard, rank,
                                         world, static_cast<unsigned>(epoch), static_cast<unsigned long long>(limit_s * 1e9),
                                         status_word(), abort_word.data_ptr<int>(), num_sms(), stream()));
}

void nvls_all_reduce(int64_t mc_ptr, Tensor local, std::vector<int64_t> flags, Tensor out, int64_t rank, int64_t world,
                     int64_t epoch, double limit_s, Tensor abort_word) {
  c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_contiguous() && local.is_contiguous() && local.scalar_type() == at::kByte &&
                  local.numel() >= out.numel() * out.element_size(), "nvls_all_reduce: contiguous output, byte view of the symmetric buffer");
  TORCH_CHECK(mc_ptr != 0, "nvls_all_reduce: no multicast address");
  FERRL_CHECK(ferrl::nvls_all_reduce(dt(out), reinterpret_cast<void*>(mc_ptr), local.data_ptr(), table_of(flags), out.data_ptr(),
                                     out.numel() * out.element_size(), rank, world, static_cast<unsigned>(epoch),
                                     static_cast<unsigned long long>(limit_s * 1e9), status_word(), abort_word.data_ptr<int>(),
                                     num_sms(), stream()));
}

int64_t launches() { return ferrl::launch_count(); }
void add_launches(int64_t n) { ferrl::count_launch(static_cast<int>(n)); }

}  // namespace

TORCH_LIBRARY(ferrl_b200, m) {
  m.def("gemm(Tensor A, Tensor B, Tensor? A2, Tensor? B2, Tensor? residual, bool out_f32, int force_bn, int force_split, int two_cta=0, Tensor? debug=None, int cluster_k=0, int stream_k=0, bool static_b=False) -> Tensor", &gemm);  // two_cta: 0 auto, -1 never, 128/256 forced
  m.def("decode_gemm(Tensor A, Tensor B, Tensor? residual=None, int glu_act=-1, int max_clusters=0, bool static_b=False, Tensor? debug=None) -> Tensor", &decode_gemm);
  m.def("set_decode_gemm(bool on) -> ()", &set_decode_gemm);
  m.def("gemm_allreduce(Tensor A, Tensor B, Tensor? A2, Tensor? B2, Tensor? residual, int[] stage, int[] outbuf, int[] flags, int rank, int world, int epoch, int max_tiles, int stage_elems, int out_elems, float limit_s, Tensor? debug=None, int mc_stage=0, int mc_outbuf=0, bool scatter=False) -> Tensor", &gemm_allreduce);
  m.def("gemm_allgather(Tensor B, Tensor? A2, Tensor? B2, int[] src, int[] flags, int rank, int world, int max_tiles, int M, int K, float limit_s) -> Tensor", &gemm_allgather);
  m.def("lora_grad(Tensor U, Tensor X) -> Tensor", &lora_grad);
  m.def("gdn_conv_fwd(Tensor x, Tensor w, Tensor? left, bool act) -> Tensor", &gdn_conv_fwd);
  m.def("gdn_conv_bwd(Tensor x, Tensor w, Tensor? left, Tensor dy, bool act) -> Tensor", &gdn_conv_bwd);
  m.def("gdn_conv_step(Tensor x, Tensor w, Tensor(a!) state, bool act) -> Tensor", &gdn_conv_step);
  m.def("gdn_chunk_fwd(Tensor q, Tensor k, Tensor v, Tensor g, Tensor beta, Tensor? S0, bool l2norm, float eps) -> (Tensor, Tensor)", &gdn_chunk_fwd);
  m.def("set_canary(bool on) -> ()", &set_canary);
  m.def("check_canaries() -> int", &check_canaries);
  m.def("rmsnorm_gated_bwd(Tensor x, Tensor gate, Tensor w, Tensor dy, float eps) -> (Tensor, Tensor)", &rmsnorm_gated_bwd);
  m.def("gdn_tc_fwd(Tensor q, Tensor k, Tensor v, Tensor g, Tensor beta, Tensor? S0) -> Tensor[]", &gdn_tc_fwd);
  m.def("gdn_tc_bwd(Tensor q, Tensor k, Tensor v, Tensor beta, Tensor Gc, Tensor gl, Tensor Tm, Tensor Wn, Tensor Kd, Tensor Vn, Tensor Sin, Tensor dO, Tensor? dS_final) -> Tensor[]", &gdn_tc_bwd);
  m.def("gdn_decode_step_raw(Tensor q, Tensor k, Tensor v, Tensor a, Tensor b, Tensor A_log, Tensor dt_bias, Tensor(a!) S, bool l2norm, float eps) -> Tensor", &gdn_decode_step_raw);
  m.def("gdn_decode_step(Tensor q, Tensor k, Tensor v, Tensor g, Tensor beta, Tensor(a!) S, bool l2norm, float eps) -> Tensor", &gdn_decode_step);
  m.def("moe_route(Tensor logits, int k, bool renorm) -> (Tensor, Tensor, Tensor, Tensor)", &moe_route);
  m.def("moe_plan(Tensor idx, Tensor counts) -> (Tensor, Tensor, Tensor, Tensor)", &moe_plan);
  m.def("moe_gather(Tensor x, Tensor token_of, Tensor? pair_w, Tensor row_of) -> Tensor", &moe_gather);
  m.def("moe_grouped_gemm(Tensor xs, Tensor W, Tensor tile_expert, Tensor(a!)? out=None) -> Tensor(a!)", &moe_grouped_gemm);
  m.def("ep_dispatch(Tensor x, Tensor idx, Tensor? pair_w, Tensor counts, int[] counts_all, int[] xs, int[] flags, int rank, int world, int epoch, float limit_s, int cap_rows, Tensor(a!) dest_row, Tensor(b!) tile_expert, Tensor(c!) local_rows, bool reuse_plan, Tensor(d!) abort_word) -> ()", &ep_dispatch);
  m.def("ep_combine(int[] ys, Tensor idx, Tensor dest_row, Tensor? w, int H, int E_local, int[] flags, int rank, int world, int epoch, float limit_s, Tensor(a!)? keep_rows, Tensor(b!) abort_word) -> Tensor", &ep_combine);
  m.def("moe_combine(Tensor ys, Tensor row_of, Tensor? w, int T, int k) -> Tensor", &moe_combine);
  m.def("moe_pair_dot(Tensor dy, Tensor ys, Tensor row_of, int k) -> Tensor", &moe_pair_dot);
  m.def("kernel_status() -> int", &kernel_status);
  m.def("reset_status() -> ()", &reset_status);
  m.def("rmsnorm(Tensor x, Tensor? res, Tensor? w, Tensor? gate, float eps, bool zc) -> (Tensor, Tensor)", &rmsnorm);
  m.def("rmsnorm_bwd(Tensor x, Tensor? w, Tensor dy, float eps, bool zc) -> Tensor", &rmsnorm_bwd);
  m.def("qk_norm_rope_fwd(Tensor q, Tensor k, Tensor? qw, Tensor? kw, Tensor cos, Tensor sin, Tensor pos, int pos_div, float eps, bool zc) -> (Tensor, Tensor)", &qk_norm_rope_fwd);
  m.def("qk_norm_rope_bwd(Tensor q, Tensor k, Tensor? qw, Tensor? kw, Tensor cos, Tensor sin, Tensor pos, int pos_div, float eps, bool zc, Tensor dq, Tensor dk, Tensor(a!) dq_in, Tensor(b!) dk_in) -> ()", &qk_norm_rope_bwd);
  m.def("kv_append(Tensor k, Tensor v, Tensor(a!) kc, Tensor(b!) vc, Tensor kv_len) -> ()", &kv_append);
  m.def("kv_append_paged(Tensor k, Tensor v, Tensor(a!) kc, Tensor(b!) vc, Tensor kv_len, Tensor table) -> ()", &kv_append_paged);
  m.def("glu_fwd(Tensor gu, int act) -> Tensor", &glu_fwd);
  m.def("glu_bwd(Tensor gu, Tensor dout, int act) -> Tensor", &glu_bwd);
  m.def("embedding(Tensor ids, Tensor table, float scale) -> Tensor", &embedding);
  m.def("lora_merge(Tensor w, Tensor a, Tensor b) -> Tensor", &lora_merge);
  m.def("adamw_step(Tensor[] params, Tensor[] grads, Tensor[] m, Tensor[] v, float lr, float b1, float b2, float eps, float wd, int step, float max_norm, float pre_scale, bool compute_norm) -> Tensor", &adamw_step);
  m.def("grpo_loss_rows(Tensor logp, Tensor logp_old, Tensor? logp_ref, Tensor adv, Tensor mask, Tensor? tis, float eps_lo, float eps_hi, float beta, bool seq_level, bool want_grad) -> (Tensor, Tensor, Tensor)", &grpo_loss_rows);
  m.def("grpo_scale_rows(Tensor(a!) dlogp, Tensor row_scale) -> ()", &grpo_scale_rows);
  m.def("decode_attn(Tensor q, Tensor kc, Tensor vc, Tensor kv_len, float scale, int window, int n_splits, Tensor? block_table, int page, int variant=0, Tensor? prefix_len=None, int group=1, int prefix_splits=1) -> Tensor", &decode_attn);
  m.def("gemm_norm(Tensor A, Tensor B, Tensor? residual, Tensor? ss_in, float eps, int glu_act, bool want_ss, bool static_b=True) -> (Tensor, Tensor)", &gemm_norm);
  m.def("row_sumsq(Tensor x) -> Tensor", &row_sumsq);
  m.def("gemm_glu(Tensor A, Tensor B, int act, bool static_b=False) -> Tensor", &gemm_glu);
  m.def("qk_norm_rope_append(Tensor q, Tensor k, Tensor v, Tensor? qw, Tensor? kw, Tensor cos_t, Tensor sin_t, Tensor pos, float eps, bool zc, Tensor(a!) kc, Tensor(b!) vc, Tensor kv_len, Tensor? table) -> Tensor", &qk_norm_rope_append);
  m.def("flash_fwd(Tensor q, Tensor k, Tensor v, float scale, bool causal, int window, int q_offset, int variant=0) -> (Tensor, Tensor)", &flash_fwd);
  m.def("flash_bwd(Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, Tensor d_o, float scale, bool causal, int window, int q_offset, int variant=0, Tensor? debug=None) -> (Tensor, Tensor, Tensor)", &flash_bwd);
  m.def("logprob_head_fwd(Tensor hidden, Tensor w, Tensor targets, float temperature, float softcap) -> (Tensor, Tensor)", &logprob_head_fwd);
  m.def("logprob_head_shard_stats(Tensor hidden, Tensor w, Tensor targets, float temperature, float softcap, int col0) -> Tensor", &logprob_head_shard_stats);
  m.def("logprob_head_dlogits(Tensor hidden, Tensor w, Tensor targets, Tensor lse, Tensor coef, float temperature, float softcap, int col0) -> Tensor", &logprob_head_dlogits);
  m.def("logprob_rows(Tensor logits, Tensor targets, float temperature, float softcap) -> (Tensor, Tensor)", &logprob_rows);
  m.def("logprob_rows_bwd(Tensor(a!) logits, Tensor targets, Tensor lse, Tensor dlp, float temperature, float softcap) -> ()", &logprob_rows_bwd);
  m.def("sample_rows(Tensor logits, Tensor global_rows, int seed, Tensor? draw_dev, int draw, float temperature, float top_p) -> (Tensor, Tensor)", &sample_rows);
  m.def("symm_alloc(int nbytes) -> Tensor", &symm_alloc);
  m.def("symm_handle(Tensor buf) -> Tensor", &symm_handle);
  m.def("symm_open(Tensor handle) -> int", &symm_open);
  m.def("symm_close(int ptr) -> ()", &symm_close);
  m.def("dp_step(int[] grads, int[] reduced, int[] flags, int[] scalars, int rank, int world, int barrier_world, int own_lo, int own_hi, int n, int epoch, float pre_scale, float uncovered_local, Tensor tables, int off_blk_tensor, int off_blk_off, int off_blk_flat, int n_blocks, int chunk, float lr, float b1, float b2, float eps, float wd, int step, float max_norm, Tensor(a!) block_partials, Tensor(b!) out, Tensor(c!) abort_word, float limit_s) -> ()", &dp_step);
  m.def("dp_tables(Tensor[] params, Tensor[] m, Tensor[] v, int[] flat_off, int chunk) -> (Tensor, int, int, int, int)", &dp_tables);
  m.def("symm_row_collective(int which, int[] src, int[] flags, Tensor(a!) out, int n_shard, int rank, int world, int epoch, float limit_s, Tensor(b!) abort_word) -> ()", &symm_row_collective);
  m.def("nvls_all_reduce(int mc_ptr, Tensor local, int[] flags, Tensor(a!) out, int rank, int world, int epoch, float limit_s, Tensor(b!) abort_word) -> ()", &nvls_all_reduce);
  m.def("symm_all_reduce(int[] src, int[] flags, Tensor(a!) out, int rank, int world, int epoch, float limit_s, Tensor(b!) abort_word) -> ()", &symm_all_reduce);
  m.def("launches() -> int", &launches);
  m.def("add_launches(int n) -> ()", &add_launches);
}
