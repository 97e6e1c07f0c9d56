// Python bindings (module superscaler_b200._C): thin, allocation-light wrappers that check
// shapes / dtypes, pick the current CUDA stream and call the kernel launchers.  Every launcher
// returns 0 or an error code; a non-zero code raises, so a missing or failing native path is
// never silent.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "attention_sm100.cuh"
#include "gemm_sm100.cuh"
#include "gemm_ar_sm100.cuh"
#include "gemm_ag_sm100.cuh"

namespace ssb {
int gemm_bf16_launch(const void* A, int lda, int a_mn_major, const void* B, int ldb, int b_mn_major,
                     const GemmParams& p, int num_sms, cudaStream_t stream);
void gemm_set_pair_mode(int mode);
int gemm_get_pair_mode();
int layernorm_fwd_launch(const void* x, const void* residual, const float* gamma, const float* beta, void* y,
                         void* sum_out, float* mean, float* rstd, int rows, int H, float eps, int num_sms,
                         cudaStream_t stream);
int ln_bwd_slices(int rows);
int ln_bwd_part_rows(int rows, int H, int num_sms);
int layernorm_bwd_launch(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                         const void* dres, void* dx, float* dgamma, float* dbeta, float* part_g, float* part_b,
                         int accumulate_wgrad, int rows, int H, int num_sms, cudaStream_t stream);
int colsum_tickets();
int colsum_launch(const void* a, int lda, float* out, float* part, int* tickets, int accumulate, int rows, int N,
                  cudaStream_t stream);
int elementwise_launch(int op, const void* x, const void* a, const void* bias, void* out, long long rows, int N,
                       float dropout_p, unsigned long long seed, int num_sms, cudaStream_t stream);
int cast_f32_to_bf16_launch(const float* in, void* out, long long n, int num_sms, cudaStream_t stream);
int softmax_fwd_launch(const void* x, const void* mask, void* y, long long rows, int sq, int sk, int heads,
                       int mask_broadcast_batch, float scale, int mode, int num_sms, cudaStream_t stream);
int softmax_bwd_launch(const void* g, const void* y, void* dx, long long rows, int sk, float scale, int num_sms,
                       cudaStream_t stream);
int sumsq_launch(const float* g, long long n, float* partials, float* out, int accumulate, cudaStream_t stream);
int adam_launch(float* p, float* m, float* v, float* g, void* p16, long long n, const float* sumsq, int* skipped,
                float lr, float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale,
                float max_norm, long long wd_end, int zero_grad, int num_sms, cudaStream_t stream);
int sgd_launch(float* p, float* mom, float* g, void* p16, long long n, const float* sumsq, int* skipped, float lr,
               float momentum, float weight_decay, float grad_scale, float max_norm, long long wd_end, int zero_grad,
               int first_step, int num_sms, cudaStream_t stream);
int embedding_fwd_launch(const long long* ids, const long long* pos, const void* W, const void* P, void* out,
                         long long tokens, int H, long long v0, long long v1, float dropout_p,
                         unsigned long long seed, int num_sms, cudaStream_t stream);
int embedding_bwd_launch(const long long* ids, const long long* pos, const void* g, float* dW, float* dP,
                         long long tokens, int H, long long v0, long long v1, float dropout_p,
                         unsigned long long seed, int num_sms, cudaStream_t stream);
int embedding_bwd_sorted_launch(const long long* keys, const long long* order, const void* g, float* dst,
                                long long tokens, int H, long long k0, long long k1, float dropout_p,
                                unsigned long long seed, cudaStream_t stream);
int ce_stats_launch(const void* logits, int ld, const long long* targets, float* row_max, float* row_sum,
                    float* row_tgt, long long rows, int V, long long v0, cudaStream_t stream);
int ce_finalize_launch(void* logits, int ld, const long long* targets, const float* gmax, const float* gsum,
                       const float* gtgt, const float* loss_mask, float* loss, long long rows, int V, long long v0,
                       float grad_scale, int write_grad, cudaStream_t stream);
int attn_fwd_launch(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const AttnParams& p,
                    cudaStream_t stream);
int attn_bwd_launch(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const void* dout,
                    int lddo, const AttnParams& p, float* delta_scratch, cudaStream_t stream);
long long attn_bwd_fused_scratch_floats(int B, int NH, int SQ, int HD);
int attn_bwd_fused_launch(const void* q, int ldq, const void* k, int ldk, const void* v, int ldv, const void* dout,
                          int lddo, const AttnParams& p, float* scratch, cudaStream_t stream);
int comm_max_blocks();
void comm_set_peer_timeout_ns(unsigned long long ns);
int allreduce_scale_f32_launch(void* const* peer_ptrs, void* mc_ptr, void* const* flag_ptrs, int rank, int world,
                               long long n, float scale, unsigned epoch, int* status, cudaStream_t stream);
int reduce_scatter_scale_sumsq_f32_launch(void* const* peer_ptrs, void* mc_ptr, void* const* flag_ptrs, int rank,
                                          int world, long long n, float scale, unsigned epoch, float* partials,
                                          int* status, cudaStream_t stream);
int allgather_b16_launch(void* const* peer_ptrs, void* mc_ptr, void* const* flag_ptrs, int rank, int world,
                         long long n, unsigned epoch, int* status, cudaStream_t stream);
void comm_slice_of(long long n_units, int world, int rank, long long* lo, long long* hi);
int bn_slices(long long rows);
int im2col_launch(const void* x, void* cols, int N, int H, int W, int C, int KH, int KW, int stride, int pad, int Kpad,
                  int num_sms, cudaStream_t stream);
int col2im_launch(const void* dcols, void* dx, int N, int H, int W, int C, int KH, int KW, int stride, int pad, int Kpad,
                  int num_sms, cudaStream_t stream);
int subsample_launch(const void* in, void* out, int N, int H, int W, int C, int stride, int scatter, int num_sms,
                     cudaStream_t stream);
int bn_fwd_launch(const void* x, const void* residual, const float* gamma, const float* beta, void* y, float* mean,
                  float* rstd, float* run_mean, float* run_var, float* part, long long rows, int C, float eps,
                  float momentum, int relu, int num_sms, cudaStream_t stream);
int bn_bwd_launch(const void* dy, const void* x, const void* y, const float* mean, const float* rstd,
                  const float* gamma, void* dx, void* dres, float* dgamma, float* dbeta, float* part, float* sums,
                  int accumulate, long long rows, int C, int relu, int num_sms, cudaStream_t stream);
int bn_apply_launch(const void* x, const void* residual, const float* mean, const float* rstd, const float* gamma,
                    const float* beta, void* y, long long rows, int C, int relu, int num_sms, cudaStream_t stream);
int maxpool_fwd_launch(const void* x, void* y, void* idx, int N, int H, int W, int C, int num_sms, cudaStream_t stream);
int maxpool_bwd_launch(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, int num_sms,
                       cudaStream_t stream);
int avgpool_launch(const void* in, void* out, int N, int HW, int C, int backward, int num_sms, cudaStream_t stream);
}  // namespace ssb

namespace {

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int num_sms() {
  static int n[64] = {0};
  int dev = at::cuda::current_device();
  if (n[dev] == 0) n[dev] = at::cuda::getDeviceProperties(dev)->multiProcessorCount;
  return n[dev];
}

// One status word per device, written by kernels whose bounded waits run out.
Tensor& status_tensor() {
  static std::vector<Tensor> st(64);
  int dev = at::cuda::current_device();
  if (!st[dev].defined()) st[dev] = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, dev));
  return st[dev];
}

// Zero-initialised ticket counters of the one-launch column sum (one set per device; every call leaves them zero).
Tensor& ticket_tensor() {
  static std::vector<Tensor> st(64);
  int dev = at::cuda::current_device();
  if (!st[dev].defined())
    st[dev] = torch::zeros({ssb::colsum_tickets()}, torch::dtype(torch::kInt32).device(torch::kCUDA, dev));
  return st[dev];
}

void check_launch(int rc, const char* what) { TORCH_CHECK(rc == 0, what, ": native launcher failed with code ", rc); }

void check_bf16_2d(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16, name, " must be a CUDA bf16 tensor");
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, " must be 2-D with unit inner stride");
}

const void* opt_ptr(const OptTensor& t) { return t.has_value() ? t->data_ptr() : nullptr; }

// D = epilogue(alpha * A op B); see gemm_sm100.cuh for the operand conventions.
void gemm(const Tensor& a, const Tensor& b, Tensor& d, bool a_mn, bool b_mn, const OptTensor& bias, int64_t act,
          const OptTensor& aux, const OptTensor& preact_out, const OptTensor& residual, bool accumulate, double alpha,
          double dropout_p, int64_t seed) {
  check_bf16_2d(a, "a");
  check_bf16_2d(b, "b");
  TORCH_CHECK(d.is_cuda() && d.dim() == 2 && d.stride(1) == 1, "d must be 2-D with unit inner stride");
  TORCH_CHECK(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32, "d must be bf16 or fp32");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm: reduction sizes differ: ", K, " vs ", Kb);
  TORCH_CHECK(d.size(0) == M && d.size(1) == N, "gemm: output must be [", M, ", ", N, "]");
  ssb::GemmParams p{};
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.D = d.data_ptr(); p.ldd = static_cast<int>(d.stride(0));
  p.out_fp32 = d.scalar_type() == torch::kFloat32;
  p.accumulate = accumulate; p.alpha = static_cast<float>(alpha);
  if (bias.has_value()) {
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "bias must be contiguous [N]");
    TORCH_CHECK(bias->scalar_type() == torch::kBFloat16 || bias->scalar_type() == torch::kFloat32, "bias dtype");
    p.bias = bias->data_ptr(); p.bias_fp32 = bias->scalar_type() == torch::kFloat32;
  }
  p.act = static_cast<int>(act);
  if (aux.has_value()) { check_bf16_2d(*aux, "aux"); p.aux = aux->data_ptr(); p.ldaux = static_cast<int>(aux->stride(0)); }
  TORCH_CHECK(!(act == ssb::kActDGelu || act == ssb::kActDRelu) || aux.has_value(), "derivative epilogues need aux");
  if (preact_out.has_value()) {
    check_bf16_2d(*preact_out, "preact_out");
    p.preact_out = preact_out->data_ptr(); p.ldpre = static_cast<int>(preact_out->stride(0));
  }
  if (residual.has_value()) {
    check_bf16_2d(*residual, "residual");
    p.residual = residual->data_ptr(); p.ldres = static_cast<int>(residual->stride(0));
  }
  for (const OptTensor* t : {&aux, &preact_out, &residual})
    if (t->has_value()) TORCH_CHECK((*t)->size(0) == M && (*t)->size(1) == N && (*t)->stride(0) % 8 == 0, "epilogue operand shape");
  p.dropout_p = static_cast<float>(dropout_p);
  p.dropout_seed = static_cast<unsigned long long>(seed);
  TORCH_CHECK(dropout_p == 0.0 || d.stride(0) == N, "dropout epilogue needs a dense output");
  p.status = status_tensor().data_ptr<int>();
  Tensor split_ws;
  const bool plain = p.out_fp32 && alpha == 1.0 && !bias.has_value() && act == 0 && !aux.has_value() &&
                     !preact_out.has_value() && !residual.has_value() && dropout_p == 0.0;
  if (plain) {
    const int splits = ssb::gemm_splitk_splits(p.M, p.N, p.K, num_sms());
    if (splits > 1) {
      split_ws = torch::empty({splits, M, N}, torch::dtype(torch::kFloat32).device(a.device()));
      p.k_splits = splits;
      p.split_ws = split_ws.data_ptr<float>();
    }
  }
  check_launch(ssb::gemm_bf16_launch(a.data_ptr(), static_cast<int>(a.stride(0)), a_mn, b.data_ptr(),
                                     static_cast<int>(b.stride(0)), b_mn, p, num_sms(), cur_stream()),
               "gemm");
}

std::vector<Tensor> layernorm_fwd(const Tensor& x, const OptTensor& residual, const Tensor& gamma, const Tensor& beta,
                                  double eps) {
  check_bf16_2d(x, "x");
  TORCH_CHECK(x.is_contiguous() && gamma.scalar_type() == torch::kFloat32 && beta.scalar_type() == torch::kFloat32);
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = static_cast<int>(x.size(0)), H = static_cast<int>(x.size(1));
  Tensor y = torch::empty_like(x);
  Tensor sum_out;
  if (residual.has_value()) { TORCH_CHECK(residual->is_contiguous() && residual->sizes() == x.sizes()); sum_out = torch::empty_like(x); }
  auto fopt = torch::dtype(torch::kFloat32).device(x.device());
  Tensor mean = torch::empty({rows}, fopt), rstd = torch::empty({rows}, fopt);
  check_launch(ssb::layernorm_fwd_launch(x.data_ptr(), opt_ptr(residual), gamma.data_ptr<float>(), beta.data_ptr<float>(),
                                         y.data_ptr(), sum_out.defined() ? sum_out.data_ptr() : nullptr,
                                         mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, H,
                                         static_cast<float>(eps), num_sms(), cur_stream()),
               "layernorm_fwd");
  if (sum_out.defined()) return {y, mean, rstd, sum_out};
  return {y, mean, rstd};
}

Tensor layernorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& gamma, const Tensor& mean, const Tensor& rstd,
                     const OptTensor& dres, Tensor& dgamma, Tensor& dbeta, bool accumulate) {
  check_bf16_2d(dy, "dy"); check_bf16_2d(x, "x");
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous());
  TORCH_CHECK(dgamma.scalar_type() == torch::kFloat32 && dbeta.scalar_type() == torch::kFloat32);
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = static_cast<int>(x.size(0)), H = static_cast<int>(x.size(1));
  Tensor dx = torch::empty_like(x);
  Tensor part = torch::empty({2, ssb::ln_bwd_part_rows(rows, H, num_sms()), H},
                             torch::dtype(torch::kFloat32).device(x.device()));
  check_launch(ssb::layernorm_bwd_launch(dy.data_ptr(), x.data_ptr(), gamma.data_ptr<float>(), mean.data_ptr<float>(),
                                         rstd.data_ptr<float>(), opt_ptr(dres), dx.data_ptr(), dgamma.data_ptr<float>(),
                                         dbeta.data_ptr<float>(), part[0].data_ptr<float>(), part[1].data_ptr<float>(),
                                         accumulate, rows, H, num_sms(), cur_stream()),
               "layernorm_bwd");
  return dx;
}

void colsum(const Tensor& a, Tensor& out, bool accumulate) {
  check_bf16_2d(a, "a");
  TORCH_CHECK(out.scalar_type() == torch::kFloat32 && out.numel() == a.size(1) && out.is_contiguous());
  c10::cuda::CUDAGuard guard(a.device());
  const int rows = static_cast<int>(a.size(0)), N = static_cast<int>(a.size(1));
  Tensor part = torch::empty({ssb::ln_bwd_slices(rows), N}, torch::dtype(torch::kFloat32).device(a.device()));
  check_launch(ssb::colsum_launch(a.data_ptr(), static_cast<int>(a.stride(0)), out.data_ptr<float>(),
                                  part.data_ptr<float>(), ticket_tensor().data_ptr<int>(), accumulate, rows, N,
                                  cur_stream()),
               "colsum");
}

Tensor elementwise(int64_t op, const Tensor& x, const OptTensor& a, const OptTensor& bias, double dropout_p,
                   int64_t seed) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous());
  if (a.has_value()) TORCH_CHECK(a->is_contiguous() && a->numel() == x.numel() && a->scalar_type() == torch::kBFloat16);
  c10::cuda::CUDAGuard guard(x.device());
  const int N = static_cast<int>(x.size(-1));
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == torch::kBFloat16 && bias->numel() == N && bias->is_contiguous());
  Tensor out = torch::empty_like(x);
  check_launch(ssb::elementwise_launch(static_cast<int>(op), x.data_ptr(), opt_ptr(a), opt_ptr(bias), out.data_ptr(),
                                       x.numel() / N, N, static_cast<float>(dropout_p),
                                       static_cast<unsigned long long>(seed), num_sms(), cur_stream()),
               "elementwise");
  return out;
}

void cast_f32_to_bf16(const Tensor& in, Tensor& out) {
  TORCH_CHECK(in.scalar_type() == torch::kFloat32 && out.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(in.is_contiguous() && out.is_contiguous() && in.numel() == out.numel());
  c10::cuda::CUDAGuard guard(in.device());
  check_launch(ssb::cast_f32_to_bf16_launch(in.data_ptr<float>(), out.data_ptr(), in.numel(), num_sms(), cur_stream()),
               "cast");
}

// x: [..., sq, sk] bf16 contiguous.  mode 0 plain, 1 causal, 2 masked (mask uint8 [b|1, 1, sq, sk]).
Tensor softmax_fwd(const Tensor& x, const OptTensor& mask, double scale, int64_t mode, int64_t heads) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() >= 2);
  c10::cuda::CUDAGuard guard(x.device());
  const int sk = static_cast<int>(x.size(-1)), sq = static_cast<int>(x.size(-2));
  const long long rows = x.numel() / sk;
  int bcast = 1;
  if (mode == 2) {
    TORCH_CHECK(mask.has_value() && mask->scalar_type() == torch::kUInt8 && mask->is_contiguous());
    bcast = mask->numel() == static_cast<int64_t>(sq) * sk;
  }
  Tensor y = torch::empty_like(x);
  check_launch(ssb::softmax_fwd_launch(x.data_ptr(), opt_ptr(mask), y.data_ptr(), rows, sq, sk, static_cast<int>(heads),
                                       bcast, static_cast<float>(scale), static_cast<int>(mode), num_sms(), cur_stream()),
               "softmax_fwd");
  return y;
}

Tensor softmax_bwd(const Tensor& g, const Tensor& y, double scale) {
  TORCH_CHECK(g.is_contiguous() && y.is_contiguous() && g.scalar_type() == torch::kBFloat16 && y.scalar_type() == torch::kBFloat16);
  c10::cuda::CUDAGuard guard(g.device());
  const int sk = static_cast<int>(g.size(-1));
  Tensor dx = torch::empty_like(g);
  check_launch(ssb::softmax_bwd_launch(g.data_ptr(), y.data_ptr(), dx.data_ptr(), g.numel() / sk, sk,
                                       static_cast<float>(scale), num_sms(), cur_stream()),
               "softmax_bwd");
  return dx;
}

void sumsq(const Tensor& g, Tensor& out, bool accumulate) {
  TORCH_CHECK(g.scalar_type() == torch::kFloat32 && g.is_contiguous() && out.scalar_type() == torch::kFloat32);
  c10::cuda::CUDAGuard guard(g.device());
  Tensor part = torch::empty({1024}, torch::dtype(torch::kFloat32).device(g.device()));
  check_launch(ssb::sumsq_launch(g.data_ptr<float>(), g.numel(), part.data_ptr<float>(), out.data_ptr<float>(),
                                 accumulate, cur_stream()),
               "sumsq");
}

void adam_step(Tensor& p, Tensor& m, Tensor& v, Tensor& g, Tensor& p16, const OptTensor& sumsq_t, const OptTensor& skipped,
               double lr, double beta1, double beta2, double eps, double wd, int64_t step, double grad_scale,
               double max_norm, int64_t wd_end, bool zero_grad) {
  TORCH_CHECK(p.is_contiguous() && m.is_contiguous() && v.is_contiguous() && g.is_contiguous() && p16.is_contiguous());
  TORCH_CHECK(p.scalar_type() == torch::kFloat32 && g.scalar_type() == torch::kFloat32 && p16.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(m.numel() == p.numel() && v.numel() == p.numel() && g.numel() == p.numel() && p16.numel() == p.numel());
  c10::cuda::CUDAGuard guard(p.device());
  check_launch(ssb::adam_launch(p.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), g.data_ptr<float>(),
                                p16.data_ptr(), p.numel(), sumsq_t.has_value() ? sumsq_t->data_ptr<float>() : nullptr,
                                skipped.has_value() ? skipped->data_ptr<int>() : nullptr, static_cast<float>(lr),
                                static_cast<float>(beta1), static_cast<float>(beta2), static_cast<float>(eps),
                                static_cast<float>(wd), static_cast<int>(step), static_cast<float>(grad_scale),
                                static_cast<float>(max_norm), wd_end, zero_grad, num_sms(), cur_stream()),
               "adam");
}

void sgd_step(Tensor& p, Tensor& mom, Tensor& g, Tensor& p16, const OptTensor& sumsq_t, const OptTensor& skipped,
              double lr, double momentum, double wd, double grad_scale, double max_norm, int64_t wd_end,
              bool zero_grad, bool first_step) {
  TORCH_CHECK(p.is_contiguous() && mom.is_contiguous() && g.is_contiguous() && p16.is_contiguous());
  c10::cuda::CUDAGuard guard(p.device());
  check_launch(ssb::sgd_launch(p.data_ptr<float>(), mom.data_ptr<float>(), g.data_ptr<float>(), p16.data_ptr(), p.numel(),
                               sumsq_t.has_value() ? sumsq_t->data_ptr<float>() : nullptr,
                               skipped.has_value() ? skipped->data_ptr<int>() : nullptr, static_cast<float>(lr),
                               static_cast<float>(momentum), static_cast<float>(wd), static_cast<float>(grad_scale),
                               static_cast<float>(max_norm), wd_end, zero_grad, first_step, num_sms(), cur_stream()),
               "sgd");
}

Tensor embedding_fwd(const Tensor& ids, const OptTensor& pos, const Tensor& W, const OptTensor& P, int64_t v0,
                     double dropout_p, int64_t seed) {
  TORCH_CHECK(ids.scalar_type() == torch::kInt64 && ids.is_contiguous() && W.scalar_type() == torch::kBFloat16 && W.is_contiguous());
  c10::cuda::CUDAGuard guard(W.device());
  const int H = static_cast<int>(W.size(1));
  Tensor out = torch::empty({ids.numel(), H}, W.options());
  if (P.has_value()) TORCH_CHECK(pos.has_value() && pos->numel() == ids.numel() && pos->scalar_type() == torch::kInt64 && P->is_contiguous());
  check_launch(ssb::embedding_fwd_launch(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()),
                                         pos.has_value() ? reinterpret_cast<const long long*>(pos->data_ptr<int64_t>()) : nullptr,
                                         W.data_ptr(), opt_ptr(P), out.data_ptr(), ids.numel(), H, v0, v0 + W.size(0),
                                         static_cast<float>(dropout_p), static_cast<unsigned long long>(seed), num_sms(),
                                         cur_stream()),
               "embedding_fwd");
  return out;
}

void embedding_bwd(const Tensor& ids, const OptTensor& pos, const Tensor& g, const OptTensor& dW, const OptTensor& dP,
                   int64_t v0, double dropout_p, int64_t seed) {
  TORCH_CHECK(g.scalar_type() == torch::kBFloat16 && g.is_contiguous());
  c10::cuda::CUDAGuard guard(g.device());
  const int H = static_cast<int>(g.size(-1));
  const int64_t v1 = dW.has_value() ? v0 + dW->size(0) : v0;
  if (dW.has_value()) TORCH_CHECK(dW->scalar_type() == torch::kFloat32 && dW->is_contiguous());
  if (dP.has_value()) TORCH_CHECK(dP->scalar_type() == torch::kFloat32 && dP->is_contiguous() && pos.has_value());
  check_launch(ssb::embedding_bwd_launch(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()),
                                         pos.has_value() ? reinterpret_cast<const long long*>(pos->data_ptr<int64_t>()) : nullptr,
                                         g.data_ptr(), dW.has_value() ? dW->data_ptr<float>() : nullptr,
                                         dP.has_value() ? dP->data_ptr<float>() : nullptr, ids.numel(), H, v0, v1,
                                         static_cast<float>(dropout_p), static_cast<unsigned long long>(seed), num_sms(),
                                         cur_stream()),
               "embedding_bwd");
}

// dst[key - k0] += sum of the (dropout-masked) rows of g whose key equals `key`; keys ascending, order[p] = token of keys[p]
void embedding_bwd_sorted(const Tensor& keys, const Tensor& order, const Tensor& g, const Tensor& dst, int64_t k0,
                          double dropout_p, int64_t seed) {
  TORCH_CHECK(g.scalar_type() == torch::kBFloat16 && g.is_contiguous() && g.is_cuda());
  TORCH_CHECK(keys.scalar_type() == torch::kInt64 && order.scalar_type() == torch::kInt64 && keys.is_contiguous() &&
              order.is_contiguous() && keys.numel() == order.numel() && keys.numel() * g.size(-1) == g.numel());
  TORCH_CHECK(dst.scalar_type() == torch::kFloat32 && dst.is_contiguous() && dst.size(-1) == g.size(-1));
  c10::cuda::CUDAGuard guard(g.device());
  check_launch(ssb::embedding_bwd_sorted_launch(reinterpret_cast<const long long*>(keys.data_ptr<int64_t>()),
                                                reinterpret_cast<const long long*>(order.data_ptr<int64_t>()),
                                                g.data_ptr(), dst.data_ptr<float>(), keys.numel(),
                                                static_cast<int>(g.size(-1)), k0, k0 + dst.size(0),
                                                static_cast<float>(dropout_p), static_cast<unsigned long long>(seed),
                                                cur_stream()),
               "embedding_bwd_sorted");
}

// returns [3, rows] fp32: local max, sum exp(x - max), target logit (0 when the target is not local)
Tensor ce_stats(const Tensor& logits, const Tensor& targets, int64_t v0) {
  check_bf16_2d(logits, "logits");
  TORCH_CHECK(targets.scalar_type() == torch::kInt64 && targets.is_contiguous() && targets.numel() == logits.size(0));
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor st = torch::empty({3, logits.size(0)}, torch::dtype(torch::kFloat32).device(logits.device()));
  check_launch(ssb::ce_stats_launch(logits.data_ptr(), static_cast<int>(logits.stride(0)),
                                    reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), st[0].data_ptr<float>(),
                                    st[1].data_ptr<float>(), st[2].data_ptr<float>(), logits.size(0),
                                    static_cast<int>(logits.size(1)), v0, cur_stream()),
               "ce_stats");
  return st;
}

// stats: [3, rows] (group max, group sum w.r.t. that max, group target logit).  Returns per-row loss;
// overwrites logits with d loss_sum / d logits * grad_scale when write_grad.
Tensor ce_finalize(Tensor& logits, const Tensor& targets, const Tensor& stats, const OptTensor& loss_mask, int64_t v0,
                   double grad_scale, bool write_grad) {
  check_bf16_2d(logits, "logits");
  TORCH_CHECK(stats.scalar_type() == torch::kFloat32 && stats.is_contiguous() && stats.size(0) == 3);
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor loss = torch::empty({logits.size(0)}, torch::dtype(torch::kFloat32).device(logits.device()));
  if (loss_mask.has_value()) TORCH_CHECK(loss_mask->scalar_type() == torch::kFloat32 && loss_mask->is_contiguous());
  check_launch(ssb::ce_finalize_launch(logits.data_ptr(), static_cast<int>(logits.stride(0)),
                                       reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
                                       stats[0].data_ptr<float>(), stats[1].data_ptr<float>(), stats[2].data_ptr<float>(),
                                       loss_mask.has_value() ? loss_mask->data_ptr<float>() : nullptr, loss.data_ptr<float>(),
                                       logits.size(0), static_cast<int>(logits.size(1)), v0,
                                       static_cast<float>(grad_scale), write_grad, cur_stream()),
               "ce_finalize");
  return loss;
}

ssb::AttnParams attn_params(int64_t B, int64_t NH, int64_t SQ, int64_t SK, int64_t HD, int64_t q_col0, int64_t k_col0,
                            int64_t v_col0, double scale, bool causal, const OptTensor& kv_lens, double dropout_p,
                            int64_t seed) {
  ssb::AttnParams p{};
  p.B = static_cast<int>(B); p.NH = static_cast<int>(NH); p.SQ = static_cast<int>(SQ); p.SK = static_cast<int>(SK);
  p.HD = static_cast<int>(HD);
  p.q_col0 = static_cast<int>(q_col0); p.k_col0 = static_cast<int>(k_col0); p.v_col0 = static_cast<int>(v_col0);
  p.scale = static_cast<float>(scale); p.causal = causal;
  if (kv_lens.has_value()) {
    TORCH_CHECK(kv_lens->scalar_type() == torch::kInt32 && kv_lens->numel() == B && kv_lens->is_contiguous());
    p.kv_lens = kv_lens->data_ptr<int>();
  }
  p.dropout_p = static_cast<float>(dropout_p);
  p.dropout_seed = static_cast<unsigned long long>(seed);
  p.status = status_tensor().data_ptr<int>();
  return p;
}

// q, k, v: 2-D bf16 matrices [B*S, ld] holding the heads at columns col0 + head*HD.
// Returns (O [B*SQ, NH*HD], LSE [B, NH, SQ]).
// bias_table (optional): fp32 [NH, SQ + SK - 1], added to the scaled scores as bias[head][key - query + SQ - 1].
std::vector<Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, int64_t B, int64_t NH, int64_t SQ,
                             int64_t SK, int64_t HD, int64_t q_col0, int64_t k_col0, int64_t v_col0, double scale,
                             bool causal, const OptTensor& kv_lens, double dropout_p, int64_t seed,
                             const OptTensor& bias_table) {
  check_bf16_2d(q, "q"); check_bf16_2d(k, "k"); check_bf16_2d(v, "v");
  TORCH_CHECK(q.size(0) == B * SQ && k.size(0) == B * SK && v.size(0) == B * SK, "attention: row counts");
  c10::cuda::CUDAGuard guard(q.device());
  ssb::AttnParams p = attn_params(B, NH, SQ, SK, HD, q_col0, k_col0, v_col0, scale, causal, kv_lens, dropout_p, seed);
  Tensor o = torch::empty({B * SQ, NH * HD}, q.options());
  Tensor lse = torch::empty({B, NH, SQ}, torch::dtype(torch::kFloat32).device(q.device()));
  p.O = o.data_ptr(); p.ldo = static_cast<int>(o.stride(0)); p.o_col0 = 0; p.LSE = lse.data_ptr<float>();
  if (bias_table.has_value()) {
    TORCH_CHECK(bias_table->is_cuda() && bias_table->scalar_type() == torch::kFloat32 && bias_table->is_contiguous() &&
                bias_table->numel() == NH * (SQ + SK - 1), "bias_table must be fp32 [NH, SQ + SK - 1]");
    p.bias_table = bias_table->data_ptr<float>();
  }
  check_launch(ssb::attn_fwd_launch(q.data_ptr(), static_cast<int>(q.stride(0)), k.data_ptr(), static_cast<int>(k.stride(0)),
                                    v.data_ptr(), static_cast<int>(v.stride(0)), p, cur_stream()),
               "attn_fwd");
  return {o, lse};
}

// false (default): the fused backward kernel, whose dQ is accumulated with floating-point reductions in arrival
// order; true: the dK/dV + dQ kernel pair, bitwise reproducible.
bool g_attn_bwd_deterministic = false;

// dq, dk, dv are written into caller-provided 2-D matrices (same conventions as q, k, v).
void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& lse, const Tensor& dout,
              Tensor& dq, Tensor& dk, Tensor& dv, int64_t B, int64_t NH, int64_t SQ, int64_t SK, int64_t HD,
              int64_t q_col0, int64_t k_col0, int64_t v_col0, int64_t dq_col0, int64_t dk_col0, int64_t dv_col0,
              double scale, bool causal, const OptTensor& kv_lens, double dropout_p, int64_t seed,
              const OptTensor& bias_table, const OptTensor& dbias_table) {
  check_bf16_2d(q, "q"); check_bf16_2d(k, "k"); check_bf16_2d(v, "v"); check_bf16_2d(o, "o"); check_bf16_2d(dout, "dout");
  check_bf16_2d(dq, "dq"); check_bf16_2d(dk, "dk"); check_bf16_2d(dv, "dv");
  TORCH_CHECK(o.stride(0) == dout.stride(0), "o and dout must share a layout");
  TORCH_CHECK(lse.scalar_type() == torch::kFloat32 && lse.is_contiguous());
  c10::cuda::CUDAGuard guard(q.device());
  ssb::AttnParams p = attn_params(B, NH, SQ, SK, HD, q_col0, k_col0, v_col0, scale, causal, kv_lens, dropout_p, seed);
  p.O = o.data_ptr(); p.ldo = static_cast<int>(o.stride(0)); p.o_col0 = 0;
  p.LSE = lse.data_ptr<float>();
  p.dQ = dq.data_ptr(); p.lddq = static_cast<int>(dq.stride(0)); p.dq_col0 = static_cast<int>(dq_col0);
  p.dK = dk.data_ptr(); p.lddk = static_cast<int>(dk.stride(0)); p.dk_col0 = static_cast<int>(dk_col0);
  p.dV = dv.data_ptr(); p.lddv = static_cast<int>(dv.stride(0)); p.dv_col0 = static_cast<int>(dv_col0);
  if (bias_table.has_value()) {
    TORCH_CHECK(dbias_table.has_value() && bias_table->scalar_type() == torch::kFloat32 && bias_table->is_contiguous() &&
                dbias_table->scalar_type() == torch::kFloat32 && dbias_table->is_contiguous() &&
                bias_table->numel() == NH * (SQ + SK - 1) && dbias_table->numel() == bias_table->numel(),
                "bias_table / dbias_table must be fp32 [NH, SQ + SK - 1]");
    p.bias_table = bias_table->data_ptr<float>();
    p.dbias_table = dbias_table->data_ptr<float>();
  }
  if (!g_attn_bwd_deterministic || bias_table.has_value()) {
    // one kernel, five tile products; dQ is summed over the key blocks in an fp32 scratch in arrival order
    Tensor scratch = torch::empty({ssb::attn_bwd_fused_scratch_floats(B, NH, SQ, HD)},
                                  torch::dtype(torch::kFloat32).device(q.device()));
    check_launch(ssb::attn_bwd_fused_launch(q.data_ptr(), static_cast<int>(q.stride(0)), k.data_ptr(),
                                            static_cast<int>(k.stride(0)), v.data_ptr(), static_cast<int>(v.stride(0)),
                                            dout.data_ptr(), static_cast<int>(dout.stride(0)), p,
                                            scratch.data_ptr<float>(), cur_stream()),
                 "attn_bwd_fused");
    return;
  }
  Tensor delta = torch::empty({B, NH, SQ}, torch::dtype(torch::kFloat32).device(q.device()));
  check_launch(ssb::attn_bwd_launch(q.data_ptr(), static_cast<int>(q.stride(0)), k.data_ptr(), static_cast<int>(k.stride(0)),
                                    v.data_ptr(), static_cast<int>(v.stride(0)), dout.data_ptr(),
                                    static_cast<int>(dout.stride(0)), p, delta.data_ptr<float>(), cur_stream()),
               "attn_bwd");
}

// ------------------------------ convolution / batch-norm / pooling ------------------------------
// x: NHWC bf16 [N, H, W, C] contiguous -> patch matrix [N*Ho*Wo, Kpad]
Tensor im2col(const Tensor& x, int64_t KH, int64_t KW, int64_t stride, int64_t pad, int64_t Kpad) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() == 4);
  c10::cuda::CUDAGuard guard(x.device());
  const int N = x.size(0), H = x.size(1), W = x.size(2), C = x.size(3);
  const int Ho = (H + 2 * pad - KH) / stride + 1, Wo = (W + 2 * pad - KW) / stride + 1;
  TORCH_CHECK(Kpad >= KH * KW * C && Kpad % 8 == 0);
  Tensor cols = torch::empty({static_cast<int64_t>(N) * Ho * Wo, Kpad}, x.options());
  check_launch(ssb::im2col_launch(x.data_ptr(), cols.data_ptr(), N, H, W, C, KH, KW, stride, pad, Kpad, num_sms(),
                                  cur_stream()), "im2col");
  return cols;
}

Tensor col2im(const Tensor& dcols, int64_t N, int64_t H, int64_t W, int64_t C, int64_t KH, int64_t KW, int64_t stride,
              int64_t pad) {
  TORCH_CHECK(dcols.is_cuda() && dcols.scalar_type() == torch::kBFloat16 && dcols.is_contiguous());
  c10::cuda::CUDAGuard guard(dcols.device());
  Tensor dx = torch::empty({N, H, W, C}, dcols.options());
  check_launch(ssb::col2im_launch(dcols.data_ptr(), dx.data_ptr(), N, H, W, C, KH, KW, stride, pad, dcols.size(1),
                                  num_sms(), cur_stream()), "col2im");
  return dx;
}

// scatter = false: [N,H,W,C] -> [N,ceil(H/s),ceil(W/s),C]; scatter = true: the transpose, given the full H, W
Tensor subsample(const Tensor& in, int64_t H, int64_t W, int64_t stride, bool scatter) {
  TORCH_CHECK(in.is_cuda() && in.scalar_type() == torch::kBFloat16 && in.is_contiguous() && in.dim() == 4);
  c10::cuda::CUDAGuard guard(in.device());
  const int64_t N = in.size(0), C = in.size(3);
  const int64_t Ho = (H + stride - 1) / stride, Wo = (W + stride - 1) / stride;
  Tensor out = scatter ? torch::empty({N, H, W, C}, in.options()) : torch::empty({N, Ho, Wo, C}, in.options());
  check_launch(ssb::subsample_launch(in.data_ptr(), out.data_ptr(), N, H, W, C, stride, scatter, num_sms(), cur_stream()),
               "subsample");
  return out;
}

// x: [rows, C] bf16.  Returns (y, mean, rstd).
std::vector<Tensor> bn_fwd(const Tensor& x, const OptTensor& residual, const Tensor& gamma, const Tensor& beta,
                           const OptTensor& run_mean, const OptTensor& run_var, double eps, double momentum, bool relu) {
  check_bf16_2d(x, "x");
  TORCH_CHECK(x.is_contiguous() && gamma.scalar_type() == torch::kFloat32 && beta.scalar_type() == torch::kFloat32);
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0);
  const int C = x.size(1);
  auto fopt = torch::dtype(torch::kFloat32).device(x.device());
  Tensor y = torch::empty_like(x), mean = torch::empty({C}, fopt), rstd = torch::empty({C}, fopt);
  Tensor part = torch::empty({ssb::bn_slices(rows), 2, C}, fopt);
  check_launch(ssb::bn_fwd_launch(x.data_ptr(), opt_ptr(residual), gamma.data_ptr<float>(), beta.data_ptr<float>(),
                                  y.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                                  run_mean.has_value() ? run_mean->data_ptr<float>() : nullptr,
                                  run_var.has_value() ? run_var->data_ptr<float>() : nullptr, part.data_ptr<float>(),
                                  rows, C, static_cast<float>(eps), static_cast<float>(momentum), relu, num_sms(),
                                  cur_stream()), "bn_fwd");
  return {y, mean, rstd};
}

// Inference BatchNorm: normalises with the given per-channel mean / rstd (fp32 [C]); returns y.
Tensor bn_apply(const Tensor& x, const OptTensor& residual, const Tensor& mean, const Tensor& rstd, const Tensor& gamma,
                const Tensor& beta, bool relu) {
  check_bf16_2d(x, "x");
  TORCH_CHECK(x.is_contiguous() && gamma.scalar_type() == torch::kFloat32 && beta.scalar_type() == torch::kFloat32 &&
              mean.scalar_type() == torch::kFloat32 && rstd.scalar_type() == torch::kFloat32 &&
              mean.numel() == x.size(1) && rstd.numel() == x.size(1));
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = torch::empty_like(x);
  check_launch(ssb::bn_apply_launch(x.data_ptr(), opt_ptr(residual), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                                    gamma.data_ptr<float>(), beta.data_ptr<float>(), y.data_ptr(), x.size(0),
                                    static_cast<int>(x.size(1)), relu, num_sms(), cur_stream()), "bn_apply");
  return y;
}

// Returns (dx, dresidual or undefined); dgamma / dbeta are written (or accumulated) in place.
std::vector<Tensor> bn_bwd(const Tensor& dy, const Tensor& x, const Tensor& y, const Tensor& mean, const Tensor& rstd,
                           const Tensor& gamma, Tensor& dgamma, Tensor& dbeta, bool accumulate, bool relu,
                           bool has_residual) {
  check_bf16_2d(dy, "dy"); check_bf16_2d(x, "x");
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && y.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0);
  const int C = x.size(1);
  auto fopt = torch::dtype(torch::kFloat32).device(x.device());
  Tensor dx = torch::empty_like(x);
  Tensor dres;
  if (has_residual) dres = torch::empty_like(x);
  Tensor part = torch::empty({ssb::bn_slices(rows), 2, C}, fopt), sums = torch::empty({2, C}, fopt);
  check_launch(ssb::bn_bwd_launch(dy.data_ptr(), x.data_ptr(), y.data_ptr(), mean.data_ptr<float>(),
                                  rstd.data_ptr<float>(), gamma.data_ptr<float>(), dx.data_ptr(),
                                  has_residual ? dres.data_ptr() : nullptr, dgamma.data_ptr<float>(),
                                  dbeta.data_ptr<float>(), part.data_ptr<float>(), sums.data_ptr<float>(), accumulate,
                                  rows, C, relu, num_sms(), cur_stream()), "bn_bwd");
  if (has_residual) return {dx, dres};
  return {dx};
}

std::vector<Tensor> maxpool_fwd(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && x.is_contiguous() && x.dim() == 4);
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t N = x.size(0), H = x.size(1), W = x.size(2), C = x.size(3);
  Tensor y = torch::empty({N, (H + 1) / 2, (W + 1) / 2, C}, x.options());
  Tensor idx = torch::empty({N, (H + 1) / 2, (W + 1) / 2, C}, torch::dtype(torch::kUInt8).device(x.device()));
  check_launch(ssb::maxpool_fwd_launch(x.data_ptr(), y.data_ptr(), idx.data_ptr(), N, H, W, C, num_sms(), cur_stream()),
               "maxpool_fwd");
  return {y, idx};
}

Tensor maxpool_bwd(const Tensor& dy, const Tensor& idx, int64_t H, int64_t W) {
  TORCH_CHECK(dy.is_contiguous() && idx.is_contiguous());
  c10::cuda::CUDAGuard guard(dy.device());
  const int64_t N = dy.size(0), C = dy.size(3);
  Tensor dx = torch::empty({N, H, W, C}, dy.options());
  check_launch(ssb::maxpool_bwd_launch(dy.data_ptr(), idx.data_ptr(), dx.data_ptr(), N, H, W, C, num_sms(), cur_stream()),
               "maxpool_bwd");
  return dx;
}

// forward: x [N, HW, C] -> [N, C]; backward: dy [N, C] -> [N, HW, C]
Tensor avgpool(const Tensor& in, int64_t HW, bool backward) {
  TORCH_CHECK(in.is_cuda() && in.scalar_type() == torch::kBFloat16 && in.is_contiguous());
  c10::cuda::CUDAGuard guard(in.device());
  const int64_t N = in.size(0), C = in.size(-1);
  Tensor out = backward ? torch::empty({N, HW, C}, in.options()) : torch::empty({N, C}, in.options());
  check_launch(ssb::avgpool_launch(in.data_ptr(), out.data_ptr(), N, HW, C, backward, num_sms(), cur_stream()), "avgpool");
  return out;
}

// In-place sum over the ranks of a symmetric fp32 buffer, times `scale`.  peer_ptrs / flag_ptrs: int64 device tensors
// holding the per-rank addresses; mc_ptr: multicast address or 0.  `epoch` must advance by 2 per call on every rank.
void allreduce_scale_f32(const Tensor& peer_ptrs, int64_t mc_ptr, const Tensor& flag_ptrs, int64_t rank, int64_t world,
                         int64_t n, double scale, int64_t epoch) {
  TORCH_CHECK(peer_ptrs.is_cuda() && peer_ptrs.scalar_type() == torch::kInt64 && peer_ptrs.numel() == world);
  TORCH_CHECK(flag_ptrs.is_cuda() && flag_ptrs.scalar_type() == torch::kInt64 && flag_ptrs.numel() == world);
  c10::cuda::CUDAGuard guard(peer_ptrs.device());
  check_launch(ssb::allreduce_scale_f32_launch(reinterpret_cast<void* const*>(peer_ptrs.data_ptr<int64_t>()),
                                               reinterpret_cast<void*>(mc_ptr),
                                               reinterpret_cast<void* const*>(flag_ptrs.data_ptr<int64_t>()), rank, world,
                                               n, static_cast<float>(scale), static_cast<unsigned>(epoch),
                                               status_tensor().data_ptr<int>(), cur_stream()),
               "allreduce_scale_f32");
}

// Reduce-scatter of the first n elements of a symmetric fp32 buffer (sum over the ranks, times `scale`): rank r ends
// up with slice r in its own buffer and the rest of its buffer cleared; `partials` [comm_max_blocks] receives per-block
// sums of squares of the reduced slice.  `epoch` must advance by 2 per call on every rank.
void reduce_scatter_scale_sumsq_f32(const Tensor& peer_ptrs, int64_t mc_ptr, const Tensor& flag_ptrs, int64_t rank,
                                    int64_t world, int64_t n, double scale, int64_t epoch, Tensor& partials) {
  TORCH_CHECK(peer_ptrs.is_cuda() && peer_ptrs.scalar_type() == torch::kInt64 && peer_ptrs.numel() == world);
  TORCH_CHECK(flag_ptrs.is_cuda() && flag_ptrs.scalar_type() == torch::kInt64 && flag_ptrs.numel() == world);
  TORCH_CHECK(partials.is_cuda() && partials.scalar_type() == torch::kFloat32 &&
              partials.numel() >= ssb::comm_max_blocks());
  c10::cuda::CUDAGuard guard(peer_ptrs.device());
  check_launch(ssb::reduce_scatter_scale_sumsq_f32_launch(
                   reinterpret_cast<void* const*>(peer_ptrs.data_ptr<int64_t>()), reinterpret_cast<void*>(mc_ptr),
                   reinterpret_cast<void* const*>(flag_ptrs.data_ptr<int64_t>()), rank, world, n,
                   static_cast<float>(scale), static_cast<unsigned>(epoch), partials.data_ptr<float>(),
                   status_tensor().data_ptr<int>(), cur_stream()),
               "reduce_scatter_scale_sumsq_f32");
}

// All-gather of the first n 16-bit elements of a symmetric buffer whose slice r is final on rank r.  One epoch per call.
void allgather_b16(const Tensor& peer_ptrs, int64_t mc_ptr, const Tensor& flag_ptrs, int64_t rank, int64_t world,
                   int64_t n, int64_t epoch) {
  TORCH_CHECK(peer_ptrs.is_cuda() && peer_ptrs.scalar_type() == torch::kInt64 && peer_ptrs.numel() == world);
  TORCH_CHECK(flag_ptrs.is_cuda() && flag_ptrs.scalar_type() == torch::kInt64 && flag_ptrs.numel() == world);
  c10::cuda::CUDAGuard guard(peer_ptrs.device());
  check_launch(ssb::allgather_b16_launch(reinterpret_cast<void* const*>(peer_ptrs.data_ptr<int64_t>()),
                                         reinterpret_cast<void*>(mc_ptr),
                                         reinterpret_cast<void* const*>(flag_ptrs.data_ptr<int64_t>()), rank, world, n,
                                         static_cast<unsigned>(epoch), status_tensor().data_ptr<int>(), cur_stream()),
               "allgather_b16");
}

// [lo, hi) in elements of rank `rank`'s slice of the first n elements (n a multiple of 8), as the two kernels split it.
std::vector<int64_t> comm_slice(int64_t n, int64_t world, int64_t rank) {
  long long lo = 0, hi = 0;
  ssb::comm_slice_of(n / 8, static_cast<int>(world), static_cast<int>(rank), &lo, &hi);
  return {lo * 8, hi * 8};
}

// out = bias / dropout / residual epilogue of the SUM over the tp ranks of (a . b^T), on every rank, in one kernel
// (csrc/gemm_ar_sm100.cu).  partial_ptrs / result_ptrs / flag_ptrs: int64 device tensors [tp] with every rank's
// address of the symmetric partial scratch, of this call's result buffer and of the flag table.
void gemm_allreduce(const Tensor& a, const Tensor& b, bool b_mn, Tensor& d, const OptTensor& bias,
                    const OptTensor& residual, double alpha, double dropout_p, int64_t seed, const Tensor& partial_ptrs,
                    const Tensor& result_ptrs, const Tensor& flag_ptrs, int64_t rank, int64_t tp,
                    int64_t epoch, int64_t max_tiles, int64_t capacity_elems, bool scatter,
                    int64_t wait_consumed_epoch) {
  check_bf16_2d(a, "a");
  check_bf16_2d(b, "b");
  check_bf16_2d(d, "d");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a.size(0), K = a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  const int64_t out_rows = scatter ? M / tp : M;   // reduce-scatter form: this rank keeps M / tp rows
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K, "gemm_allreduce: reduction sizes differ");
  TORCH_CHECK(!scatter || M % (tp * 128) == 0, "reduce-scatter form: rows per rank must be a multiple of 128");
  TORCH_CHECK(d.size(0) == out_rows && d.size(1) == N, "gemm_allreduce: output must be [", out_rows, ", ", N, "]");
  for (const Tensor* t : {&partial_ptrs, &result_ptrs, &flag_ptrs})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kInt64 && t->numel() == tp, "pointer tables must be int64 [tp]");
  ssb::GemmParams p{};
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.D = d.data_ptr(); p.ldd = static_cast<int>(d.stride(0));
  p.alpha = static_cast<float>(alpha);
  if (bias.has_value()) {
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "bias must be contiguous [N]");
    TORCH_CHECK(bias->scalar_type() == torch::kBFloat16 || bias->scalar_type() == torch::kFloat32, "bias dtype");
    p.bias = bias->data_ptr(); p.bias_fp32 = bias->scalar_type() == torch::kFloat32;
  }
  if (residual.has_value()) {
    check_bf16_2d(*residual, "residual");
    TORCH_CHECK(residual->size(0) == out_rows && residual->size(1) == N && residual->stride(0) % 8 == 0, "residual shape");
    p.residual = residual->data_ptr(); p.ldres = static_cast<int>(residual->stride(0));
  }
  p.dropout_p = static_cast<float>(dropout_p);
  p.dropout_seed = static_cast<unsigned long long>(seed);
  p.status = status_tensor().data_ptr<int>();
  ssb::GemmArComm cm{};
  cm.scatter = scatter ? 1 : 0;
  cm.wait_consumed_epoch = static_cast<uint32_t>(wait_consumed_epoch);
  cm.partial_ptrs = reinterpret_cast<const void* const*>(partial_ptrs.data_ptr<int64_t>());
  cm.result_ptrs = reinterpret_cast<const void* const*>(result_ptrs.data_ptr<int64_t>());
  cm.flag_ptrs = reinterpret_cast<uint32_t* const*>(flag_ptrs.data_ptr<int64_t>());
  cm.capacity_elems = capacity_elems;

  cm.rank = static_cast<int>(rank); cm.tp = static_cast<int>(tp);
  cm.epoch = static_cast<uint32_t>(epoch); cm.max_tiles = static_cast<int>(max_tiles);
  check_launch(ssb::gemm_ar_launch(a.data_ptr(), static_cast<int>(a.stride(0)), b.data_ptr(),
                                   static_cast<int>(b.stride(0)), b_mn, p, cm, num_sms(), cur_stream()),
               "gemm_allreduce");
}

// y = epilogue(concat over the tp ranks of x_r . w^T) in one kernel (csrc/gemm_ag_sm100.cu).  x: this rank's rows
// [M / tp, K]; gather_ptrs / flag_ptrs: int64 device tensors [tp]; gather_local: this rank's gather buffer address.
void allgather_gemm(const Tensor& x, const Tensor& w, Tensor& d, const OptTensor& bias, int64_t act,
                    const OptTensor& preact_out, const Tensor& gather_ptrs, int64_t gather_local, const Tensor& flag_ptrs,
                    int64_t rank, int64_t tp, int64_t epoch, int64_t max_blocks, int64_t capacity_elems) {
  check_bf16_2d(x, "x");
  check_bf16_2d(w, "w");
  check_bf16_2d(d, "d");
  TORCH_CHECK(x.is_contiguous(), "x must be dense");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t M = x.size(0) * tp, K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K, "allgather_gemm: reduction sizes differ");
  TORCH_CHECK(d.size(0) == M && d.size(1) == N, "allgather_gemm: output must be [", M, ", ", N, "]");
  for (const Tensor* t : {&gather_ptrs, &flag_ptrs})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kInt64 && t->numel() == tp, "pointer tables must be int64 [tp]");
  ssb::GemmParams p{};
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.D = d.data_ptr(); p.ldd = static_cast<int>(d.stride(0));
  p.alpha = 1.0f;
  if (bias.has_value()) {
    TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "bias must be contiguous [N]");
    p.bias = bias->data_ptr(); p.bias_fp32 = bias->scalar_type() == torch::kFloat32;
  }
  p.act = static_cast<int>(act);
  if (preact_out.has_value()) {
    check_bf16_2d(*preact_out, "preact_out");
    TORCH_CHECK(preact_out->size(0) == M && preact_out->size(1) == N, "preact_out shape");
    p.preact_out = preact_out->data_ptr(); p.ldpre = static_cast<int>(preact_out->stride(0));
  }
  p.status = status_tensor().data_ptr<int>();
  ssb::GemmAgComm cm{};
  cm.x_local = x.data_ptr();
  cm.gather_ptrs = reinterpret_cast<void* const*>(gather_ptrs.data_ptr<int64_t>());
  cm.gather_ptrs_host_local = reinterpret_cast<const void*>(gather_local);
  cm.flag_ptrs = reinterpret_cast<uint32_t* const*>(flag_ptrs.data_ptr<int64_t>());
  cm.rank = static_cast<int>(rank); cm.tp = static_cast<int>(tp);
  cm.epoch = static_cast<uint32_t>(epoch); cm.max_blocks = static_cast<int>(max_blocks);
  cm.capacity_elems = capacity_elems;
  check_launch(ssb::gemm_ag_launch(w.data_ptr(), static_cast<int>(w.stride(0)), p, cm, num_sms(), cur_stream()),
               "allgather_gemm");
}

int64_t comm_max_blocks() { return ssb::comm_max_blocks(); }

Tensor status() { return status_tensor(); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm);
  m.def("gemm_allreduce", &gemm_allreduce);
  m.def("allgather_gemm", &allgather_gemm);
  m.def("gemm_splitk_splits", [](int64_t M, int64_t N, int64_t K) {
    return ssb::gemm_splitk_splits(static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), num_sms());
  });
  m.def("gemm_set_pair_mode", &ssb::gemm_set_pair_mode);
  m.def("gemm_get_pair_mode", &ssb::gemm_get_pair_mode);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("colsum", &colsum);
  m.def("elementwise", &elementwise);
  m.def("cast_f32_to_bf16", &cast_f32_to_bf16);
  m.def("softmax_fwd", &softmax_fwd);
  m.def("softmax_bwd", &softmax_bwd);
  m.def("sumsq", &sumsq);
  m.def("adam_step", &adam_step);
  m.def("sgd_step", &sgd_step);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("embedding_bwd_sorted", &embedding_bwd_sorted);
  m.def("ce_stats", &ce_stats);
  m.def("ce_finalize", &ce_finalize);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  m.def("set_attn_bwd_deterministic", [](bool on) { g_attn_bwd_deterministic = on; });
  m.def("attn_bwd_deterministic", []() { return g_attn_bwd_deterministic; });
  m.def("im2col", &im2col);
  m.def("col2im", &col2im);
  m.def("subsample", &subsample);
  m.def("bn_fwd", &bn_fwd);
  m.def("bn_bwd", &bn_bwd);
  m.def("bn_apply", &bn_apply);
  m.def("maxpool_fwd", &maxpool_fwd);
  m.def("maxpool_bwd", &maxpool_bwd);
  m.def("avgpool", &avgpool);
  m.def("allreduce_scale_f32", &allreduce_scale_f32);
  m.def("reduce_scatter_scale_sumsq_f32", &reduce_scatter_scale_sumsq_f32);
  m.def("allgather_b16", &allgather_b16);
  m.def("comm_slice", &comm_slice);
  m.def("comm_max_blocks", &comm_max_blocks);
  m.def("status", &status);
  m.def("comm_set_peer_timeout_ms", [](double ms) { ssb::comm_set_peer_timeout_ns(static_cast<unsigned long long>(ms * 1e6)); });
}
