// torch.ops.oslo_b200.*: argument checking, allocation and stream plumbing around the C launchers.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "oslo_kernels.h"

namespace {

using at::Tensor;
using c10::optional;

int dt_code(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kBFloat16: return OSLO_DT_BF16;
    case at::kHalf: return OSLO_DT_FP16;
    case at::kFloat: return OSLO_DT_FP32;
    default: TORCH_CHECK(false, "oslo_b200: unsupported dtype ", t.scalar_type());
  }
}
void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "oslo_b200::", what, " failed with code ", rc,
              rc > 0 ? std::string(" (") + cudaGetErrorString(static_cast<cudaError_t>(rc)) + ")" : std::string());
}
std::atomic<int64_t> g_launches{0};
// every binding passes through here once per kernel it enqueues
cudaStream_t cur_stream(int kernels = 1) {
  g_launches.fetch_add(kernels, std::memory_order_relaxed);
  return at::cuda::getCurrentCUDAStream().stream();
}
int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }
// SMs that the persistent GEMM kernels leave free (their grids are sized for `SM count - reserved`). A pipeline stage
// keeps point-to-point transfers in flight that wait for the neighbouring stage while holding an SM each; with a
// statically scheduled persistent grid every SM taken away would delay that SM's whole share of the tiles to the end
// of the kernel. Process-wide; every rank of a tensor-parallel group must use the same value (the fused GEMM +
// collective kernels need the same grid on every rank).
std::atomic<int> g_reserved_sms{0};
int64_t set_reserved_sms(int64_t n) {
  const int prev = g_reserved_sms.exchange(static_cast<int>(n < 0 ? 0 : n));
  return prev;
}
int64_t reserved_sms() { return g_reserved_sms.load(); }
const void* ptr_or_null(const optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

struct DevState {
  Tensor err;
  int sms = 0;
};
DevState& dev_state(int dev) {
  static std::mutex mu;
  static std::unordered_map<int, DevState> states;
  std::lock_guard<std::mutex> g(mu);
  auto it = states.find(dev);
  if (it == states.end()) {
    DevState s;
    s.err = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, dev));
    s.sms = at::cuda::getDeviceProperties(dev)->multiProcessorCount;
    it = states.emplace(dev, std::move(s)).first;
  }
  return it->second;
}

// SM count the persistent kernels may fill: all of them minus the reserved ones, an even number of at least 2
int usable_sms(const DevState& st) {
  int n = st.sms - g_reserved_sms.load(std::memory_order_relaxed);
  if (n < 2) n = 2;
  return n & ~1;
}

// The word that kernels set when a bounded wait runs out (0 = no error). Reading it synchronises.
Tensor error_word(const Tensor& like) { return dev_state(like.get_device()).err; }

void check_2d_operand(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 2, name, " must be a 2-D CUDA tensor");
  TORCH_CHECK(t.stride(1) == 1 && t.stride(0) % 8 == 0 && t.stride(0) >= t.size(1), name,
              " needs a contiguous last dim and a row stride that is a multiple of 8 elements");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, " must be 16-byte aligned");
}

// D[M,N] = alpha * A x B^T-style product with fused epilogue; see gemm_sm100.cu for the operand layouts.
Tensor gemm(const Tensor& a, const Tensor& b, int64_t a_mn, int64_t b_mn, const optional<Tensor>& bias,
            const optional<Tensor>& aux, const optional<Tensor>& out, const optional<Tensor>& aux_out, int64_t flags,
            double alpha) {
  check_2d_operand(a, "a");
  check_2d_operand(b, "b");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "a and b must share a dtype");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf, "gemm inputs must be bf16 or fp16");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "contraction sizes differ: ", K, " vs ", Kb);
  int fl = static_cast<int>(flags) & ~GEMM_FLAG_FP16;
  if (a.scalar_type() == at::kHalf) fl |= GEMM_FLAG_FP16;
  const bool out_f32 = fl & GEMM_FLAG_OUT_FP32;
  Tensor d;
  if (out.has_value() && out->defined()) {
    d = *out;
    TORCH_CHECK(d.is_cuda() && d.dim() == 2 && d.size(0) == M && d.size(1) == N && d.stride(1) == 1, "bad out");
    TORCH_CHECK(d.scalar_type() == (out_f32 ? at::kFloat : a.scalar_type()), "out dtype does not match flags");
  } else {
    TORCH_CHECK(!(fl & GEMM_FLAG_ACCUMULATE), "accumulate needs an out tensor");
    d = at::empty({M, N}, a.options().dtype(out_f32 ? at::kFloat : a.scalar_type()));
  }
  if (M == 0 || N == 0) return d;
  if (fl & GEMM_FLAG_BIAS) {
    TORCH_CHECK(bias.has_value() && bias->numel() == N && bias->scalar_type() == a.scalar_type() && bias->is_contiguous(),
                "bias must be a contiguous [N] tensor of the input dtype");
  }
  int ld_aux = 0, ld_aux_out = 0;
  if (fl & (GEMM_FLAG_DGELU | GEMM_FLAG_RESIDUAL)) {
    TORCH_CHECK(!((fl & GEMM_FLAG_DGELU) && (fl & GEMM_FLAG_RESIDUAL)), "dgelu and residual share the aux operand");
    TORCH_CHECK(aux.has_value() && aux->dim() == 2 && aux->size(0) == M && aux->size(1) == N && aux->stride(1) == 1, "bad aux");
    const auto want = (fl & GEMM_FLAG_RESIDUAL) ? d.scalar_type() : a.scalar_type();
    TORCH_CHECK(aux->scalar_type() == want, "aux dtype mismatch");
    ld_aux = static_cast<int>(aux->stride(0));
  }
  if (fl & GEMM_FLAG_SAVE_PREACT) {
    TORCH_CHECK(aux_out.has_value() && aux_out->dim() == 2 && aux_out->size(0) == M && aux_out->size(1) == N &&
                    aux_out->stride(1) == 1 && aux_out->scalar_type() == a.scalar_type(), "bad aux_out");
    ld_aux_out = static_cast<int>(aux_out->stride(0));
  }
  auto& st = dev_state(a.get_device());
  const int rc = oslo_gemm_16bit(a.data_ptr(), b.data_ptr(), d.data_ptr(), static_cast<int>(M), static_cast<int>(N),
                                 static_cast<int>(K), static_cast<int>(a.stride(0)), static_cast<int>(b.stride(0)),
                                 static_cast<int>(d.stride(0)), static_cast<int>(a_mn), static_cast<int>(b_mn),
                                 ptr_or_null(bias), ptr_or_null(aux), ld_aux,
                                 const_cast<void*>(ptr_or_null(aux_out)), ld_aux_out, fl, static_cast<float>(alpha),
                                 st.err.data_ptr<int>(), usable_sms(st), cur_stream());
  check_rc(rc, "gemm");
  return d;
}

// LM-head projection whose epilogue does the cross-entropy work; the logits a @ b^T + bias are never stored.
//   forward  (lse undefined): returns (rowmax, sumexp, target logit), fp32 [M] each
//   backward (lse, scale given): returns ((softmax - onehot) * scale) [M, N] in the input dtype, written into `out`
//   when given
std::tuple<Tensor, Tensor, Tensor> gemm_ce_stats(const Tensor& a, const Tensor& b, int64_t b_mn, const optional<Tensor>& bias,
                                                 const Tensor& labels, int64_t vocab_start) {
  check_2d_operand(a, "a");
  check_2d_operand(b, "b");
  TORCH_CHECK(a.scalar_type() == b.scalar_type() && (a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf),
              "gemm_ce inputs must both be bf16 or fp16");
  const int64_t M = a.size(0), K = a.size(1), N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K, "contraction sizes differ");
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == at::kLong && labels.numel() == M && labels.is_contiguous(), "bad labels");
  const bool has_bias = bias.has_value() && bias->defined();
  if (has_bias) TORCH_CHECK(bias->numel() == N && bias->scalar_type() == a.scalar_type() && bias->is_contiguous(), "bad bias");
  c10::cuda::CUDAGuard guard(a.device());
  auto f32 = a.options().dtype(at::kFloat);
  Tensor mx = at::empty({M}, f32), se = at::empty({M}, f32), tg = at::empty({M}, f32);
  if (M == 0) return {mx, se, tg};
  const int64_t blocks = (N + GEMM_CE_BLOCK - 1) / GEMM_CE_BLOCK;
  Tensor stats = at::empty({blocks, M, 3}, f32);
  auto& st = dev_state(a.get_device());
  check_rc(oslo_gemm_ce_16bit(a.data_ptr(), b.data_ptr(), static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
                              static_cast<int>(a.stride(0)), static_cast<int>(b.stride(0)), static_cast<int>(b_mn),
                              has_bias ? bias->data_ptr() : nullptr,
                              reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), vocab_start, 0,
                              stats.data_ptr<float>(), nullptr, nullptr, nullptr, 0, a.scalar_type() == at::kHalf ? 1 : 0,
                              st.err.data_ptr<int>(), usable_sms(st), cur_stream()), "gemm_ce_stats");
  check_rc(oslo_ce_reduce_stats(stats.data_ptr<float>(), mx.data_ptr<float>(), se.data_ptr<float>(), tg.data_ptr<float>(),
                                static_cast<int>(M), static_cast<int>(blocks), cur_stream()), "ce_reduce_stats");
  return {mx, se, tg};
}
Tensor gemm_ce_grad(const Tensor& a, const Tensor& b, int64_t b_mn, const optional<Tensor>& bias, const Tensor& labels,
                    int64_t vocab_start, const Tensor& lse, const Tensor& scale) {
  check_2d_operand(a, "a");
  check_2d_operand(b, "b");
  TORCH_CHECK(a.scalar_type() == b.scalar_type() && (a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf),
              "gemm_ce inputs must both be bf16 or fp16");
  const int64_t M = a.size(0), K = a.size(1), N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K, "contraction sizes differ");
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == at::kLong && labels.numel() == M && labels.is_contiguous(), "bad labels");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.numel() == M && lse.is_contiguous() &&
              scale.scalar_type() == at::kFloat && scale.numel() == M && scale.is_contiguous(), "lse / scale must be fp32 [M]");
  const bool has_bias = bias.has_value() && bias->defined();
  if (has_bias) TORCH_CHECK(bias->numel() == N && bias->scalar_type() == a.scalar_type() && bias->is_contiguous(), "bad bias");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor d = at::empty({M, N}, a.options());
  if (M == 0) return d;
  auto& st = dev_state(a.get_device());
  check_rc(oslo_gemm_ce_16bit(a.data_ptr(), b.data_ptr(), static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
                              static_cast<int>(a.stride(0)), static_cast<int>(b.stride(0)), static_cast<int>(b_mn),
                              has_bias ? bias->data_ptr() : nullptr,
                              reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), vocab_start, 1, nullptr,
                              lse.data_ptr<float>(), scale.data_ptr<float>(), d.data_ptr(), static_cast<int>(d.stride(0)),
                              a.scalar_type() == at::kHalf ? 1 : 0, st.err.data_ptr<int>(), usable_sms(st), cur_stream()),
           "gemm_ce_grad");
  return d;
}

// y = act(a @ b^T + bias) for few rows (decode steps): split-K GEMM into fp32 planes, then one finalisation
// kernel that sums them in a fixed order. Falls back to the ordinary GEMM when splitting the k range gains nothing.
// `gelu_from`: -1 = no activation, c >= 0 = tanh-GeLU on output columns >= c (0 = all of them), which lets one GEMM
// serve several layers that share an input when only the last of them is followed by the activation.
Tensor gemm_small_m(const Tensor& a, const Tensor& b, int64_t b_mn, const optional<Tensor>& bias, int64_t gelu_from) {
  check_2d_operand(a, "a");
  check_2d_operand(b, "b");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "a and b must share a dtype");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf, "gemm inputs must be bf16 or fp16");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a.size(0), K = a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "contraction sizes differ: ", K, " vs ", Kb);
  auto& st = dev_state(a.get_device());
  const int split = std::max(1, oslo_gemm_split_k_for(static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), usable_sms(st)));
  const bool has_bias = bias.has_value() && bias->defined();
  if (has_bias)
    TORCH_CHECK(bias->numel() == N && bias->scalar_type() == a.scalar_type() && bias->is_contiguous(), "bad bias");
  if (split <= 1 && gelu_from <= 0) {
    const int64_t fl = (has_bias ? GEMM_FLAG_BIAS : 0) | (gelu_from == 0 ? GEMM_FLAG_GELU : 0);
    return gemm(a, b, 0, b_mn, bias, optional<Tensor>(), optional<Tensor>(), optional<Tensor>(), fl, 1.0);
  }
  Tensor ws = at::empty({split, M, N}, a.options().dtype(at::kFloat));
  check_rc(oslo_gemm_splitk_16bit(a.data_ptr(), b.data_ptr(), ws.data_ptr<float>(), static_cast<int>(M),
                                  static_cast<int>(N), static_cast<int>(K), static_cast<int>(a.stride(0)),
                                  static_cast<int>(b.stride(0)), static_cast<int>(N), 0, static_cast<int>(b_mn),
                                  a.scalar_type() == at::kHalf ? 1 : 0, split, st.err.data_ptr<int>(), usable_sms(st),
                                  cur_stream()), "gemm_splitk");
  Tensor y = at::empty({M, N}, a.options());
  check_rc(oslo_splitk_finalize(ws.data_ptr<float>(), has_bias ? bias->data_ptr() : nullptr, y.data_ptr(), M,
                                static_cast<int>(N), split, static_cast<int>(gelu_from), dt_code(a), cur_stream()), "splitk_finalize");
  return y;
}

std::tuple<Tensor, Tensor, Tensor> layernorm_fwd(const Tensor& x, const Tensor& w, const optional<Tensor>& b, double eps) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && w.is_contiguous(), "layernorm: contiguous CUDA tensors required");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t cols = x.size(-1), rows = x.numel() / std::max<int64_t>(cols, 1);
  Tensor y = at::empty_like(x);
  Tensor mean = at::empty({rows}, x.options().dtype(at::kFloat));
  Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  check_rc(oslo_layernorm_fwd(x.data_ptr(), w.data_ptr(), ptr_or_null(b), y.data_ptr(), mean.data_ptr<float>(),
                              rstd.data_ptr<float>(), static_cast<int>(rows), static_cast<int>(cols),
                              static_cast<float>(eps), dt_code(x), cur_stream()), "layernorm_fwd");
  return {y, mean, rstd};
}

std::tuple<Tensor, Tensor, Tensor> layernorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& mean,
                                                  const Tensor& rstd) {
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous(), "layernorm_bwd: contiguous tensors required");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t cols = x.size(-1), rows = x.numel() / std::max<int64_t>(cols, 1);
  const int parts = static_cast<int>(std::min<int64_t>(rows, 2 * dev_state(x.get_device()).sms));
  Tensor dx = at::empty_like(x);
  Tensor dw = at::empty_like(w), db = at::empty_like(w);
  Tensor part = at::empty({2, std::max(parts, 1), cols}, x.options().dtype(at::kFloat));
  check_rc(oslo_layernorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
                              dx.data_ptr(), part[0].data_ptr<float>(), part[1].data_ptr<float>(), dw.data_ptr(),
                              db.data_ptr(), static_cast<int>(rows), static_cast<int>(cols), parts, dt_code(x),
                              cur_stream(2)), "layernorm_bwd");
  return {dx, dw, db};
}

Tensor bias_gelu_fwd(const Tensor& x, const optional<Tensor>& bias) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "bias_gelu: contiguous CUDA tensor required");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  const int64_t cols = x.size(-1);
  check_rc(oslo_bias_gelu_fwd(x.data_ptr(), ptr_or_null(bias), y.data_ptr(), x.numel() / std::max<int64_t>(cols, 1),
                              static_cast<int>(cols), dt_code(x), cur_stream()), "bias_gelu_fwd");
  return y;
}
Tensor bias_gelu_bwd(const Tensor& dy, const Tensor& x, const optional<Tensor>& bias) {
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous(), "bias_gelu_bwd: contiguous tensors required");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = at::empty_like(x);
  const int64_t cols = x.size(-1);
  check_rc(oslo_bias_gelu_bwd(dy.data_ptr(), x.data_ptr(), ptr_or_null(bias), dx.data_ptr(),
                              x.numel() / std::max<int64_t>(cols, 1), static_cast<int>(cols), dt_code(x), cur_stream()),
           "bias_gelu_bwd");
  return dx;
}

Tensor bias_dropout_residual(const Tensor& x, const optional<Tensor>& bias, const optional<Tensor>& residual, double p,
                             int64_t seed, int64_t mode) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "bias_dropout_residual: contiguous CUDA tensor required");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  const int64_t cols = x.size(-1);
  check_rc(oslo_bias_dropout_residual(x.data_ptr(), ptr_or_null(bias), ptr_or_null(residual), y.data_ptr(),
                                      x.numel() / std::max<int64_t>(cols, 1), static_cast<int>(cols),
                                      static_cast<float>(p), static_cast<unsigned long long>(seed),
                                      static_cast<int>(mode), dt_code(x), cur_stream()), "bias_dropout_residual");
  return y;
}

Tensor colsum(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous(), "colsum: contiguous 2-D CUDA tensor required");
  c10::cuda::CUDAGuard guard(x.device());
  const int rows = static_cast<int>(x.size(0)), cols = static_cast<int>(x.size(1));
  const int parts = std::max(1, std::min(rows, 64));
  Tensor part = at::empty({parts, cols}, x.options().dtype(at::kFloat));
  Tensor out = at::zeros({cols}, x.options().dtype(at::kFloat));
  check_rc(oslo_colsum(x.data_ptr(), part.data_ptr<float>(), out.data_ptr<float>(), rows, cols, parts, dt_code(x),
                       cur_stream(2)), "colsum");
  return out;
}

Tensor rotary(const Tensor& x, const Tensor& positions, int64_t rotary_dim, double base, bool inverse) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.is_contiguous(), "rotary: contiguous [B,S,H,D] CUDA tensor required");
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous() &&
                  positions.numel() == x.size(0) * x.size(1), "rotary: positions must be int64 [B,S]");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  check_rc(oslo_rotary(x.data_ptr(), y.data_ptr(), reinterpret_cast<const long long*>(positions.data_ptr<int64_t>()),
                       static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), static_cast<int>(x.size(2)),
                       static_cast<int>(x.size(3)), static_cast<int>(rotary_dim), static_cast<float>(base),
                       inverse ? 1 : 0, dt_code(x), cur_stream()), "rotary");
  return y;
}

// in place: only the first rotary_dim dims of every head are read and written. x is any contiguous tensor whose
// memory is [tokens, heads, head_dim] (e.g. the [B, S, heads * head_dim] output of a projection)
Tensor rotary_(Tensor x, const Tensor& positions, int64_t heads, int64_t head_dim, int64_t rotary_dim, double base,
               bool inverse) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "rotary_: contiguous CUDA tensor required");
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous() &&
                  positions.numel() * heads * head_dim == x.numel(), "rotary_: positions must be int64 [tokens]");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(oslo_rotary_inplace(x.data_ptr(), reinterpret_cast<const long long*>(positions.data_ptr<int64_t>()), 1,
                               static_cast<int>(positions.numel()), static_cast<int>(heads), static_cast<int>(head_dim),
                               static_cast<int>(rotary_dim), static_cast<float>(base), inverse ? 1 : 0, dt_code(x),
                               cur_stream()), "rotary_");
  return x;
}

Tensor causal_softmax_fwd(const Tensor& x, double scale) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.is_contiguous(), "causal_softmax: contiguous [batches,sq,sk] required");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  check_rc(oslo_causal_softmax_fwd(x.data_ptr(), y.data_ptr(), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)),
                                   static_cast<int>(x.size(2)), static_cast<float>(scale), dt_code(x), cur_stream()),
           "causal_softmax_fwd");
  return y;
}
Tensor masked_softmax_fwd(const Tensor& x, const Tensor& mask, double scale) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.is_contiguous(), "masked_softmax: contiguous [b,h,sq,sk] required");
  TORCH_CHECK(mask.scalar_type() == at::kByte && mask.is_contiguous() && mask.dim() == 4 && mask.size(1) == 1 &&
                  mask.size(2) == x.size(2) && mask.size(3) == x.size(3) &&
                  (mask.size(0) == 1 || mask.size(0) == x.size(0)), "mask must be uint8 [1|b,1,sq,sk]");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  check_rc(oslo_masked_softmax_fwd(x.data_ptr(), mask.data_ptr<uint8_t>(), y.data_ptr(), static_cast<int>(x.size(0)),
                                   static_cast<int>(x.size(1)), static_cast<int>(x.size(2)), static_cast<int>(x.size(3)),
                                   static_cast<int>(mask.size(0)), static_cast<float>(scale), dt_code(x), cur_stream()),
           "masked_softmax_fwd");
  return y;
}
Tensor softmax_bwd(const Tensor& y, const Tensor& dy, double scale) {
  TORCH_CHECK(y.is_contiguous() && dy.is_contiguous(), "softmax_bwd: contiguous tensors required");
  c10::cuda::CUDAGuard guard(y.device());
  Tensor dx = at::empty_like(y);
  const int64_t cols = y.size(-1);
  check_rc(oslo_softmax_bwd(y.data_ptr(), dy.data_ptr(), dx.data_ptr(), y.numel() / std::max<int64_t>(cols, 1),
                            static_cast<int>(cols), static_cast<float>(scale), dt_code(y), cur_stream()), "softmax_bwd");
  return dx;
}

std::tuple<Tensor, Tensor, Tensor> ce_stats(const Tensor& logits, const Tensor& labels, int64_t vocab_start) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "ce_stats: [rows, cols] logits required");
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == logits.size(0), "bad labels");
  c10::cuda::CUDAGuard guard(logits.device());
  const auto fo = logits.options().dtype(at::kFloat);
  Tensor mx = at::empty({logits.size(0)}, fo), se = at::empty({logits.size(0)}, fo), tg = at::empty({logits.size(0)}, fo);
  check_rc(oslo_ce_stats(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                         mx.data_ptr<float>(), se.data_ptr<float>(), tg.data_ptr<float>(), static_cast<int>(logits.size(0)),
                         static_cast<int>(logits.size(1)), static_cast<int>(logits.stride(0)), vocab_start,
                         dt_code(logits), cur_stream()), "ce_stats");
  return {mx, se, tg};
}
Tensor ce_grad_(Tensor logits, const Tensor& labels, int64_t vocab_start, const Tensor& lse, const Tensor& scale) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1, "ce_grad_: [rows, cols] logits required");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && scale.scalar_type() == at::kFloat && lse.is_contiguous() &&
                  scale.is_contiguous() && labels.is_contiguous(), "ce_grad_: fp32 contiguous lse/scale required");
  c10::cuda::CUDAGuard guard(logits.device());
  check_rc(oslo_ce_grad(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                        lse.data_ptr<float>(), scale.data_ptr<float>(), static_cast<int>(logits.size(0)),
                        static_cast<int>(logits.size(1)), static_cast<int>(logits.stride(0)), vocab_start,
                        dt_code(logits), cur_stream()), "ce_grad");
  return logits;
}

void adam_step(Tensor p, const Tensor& g, Tensor m, Tensor v, const optional<Tensor>& p_lp, double lr, double beta1,
               double beta2, double eps, double wd, int64_t step, double grad_scale, const optional<Tensor>& inv_scale) {
  TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat,
              "adam: fp32 master/moment buffers required");
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous() &&
                  g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel(), "adam: size mismatch");
  c10::cuda::CUDAGuard guard(p.device());
  int lp_dt = OSLO_DT_BF16;
  if (p_lp.has_value() && p_lp->defined()) {
    TORCH_CHECK(p_lp->is_contiguous() && p_lp->numel() == p.numel(), "adam: low-precision copy size mismatch");
    lp_dt = dt_code(*p_lp);
    TORCH_CHECK(lp_dt != OSLO_DT_FP32, "adam: low-precision copy must be 16-bit");
  }
  const float bc1 = 1.f - static_cast<float>(std::pow(beta1, static_cast<double>(step)));
  const float bc2 = 1.f - static_cast<float>(std::pow(beta2, static_cast<double>(step)));
  const float* inv = inv_scale.has_value() && inv_scale->defined() ? inv_scale->data_ptr<float>() : nullptr;
  check_rc(oslo_adam(p.data_ptr<float>(), g.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(),
                     const_cast<void*>(ptr_or_null(p_lp)), p.numel(), static_cast<float>(lr), static_cast<float>(beta1),
                     static_cast<float>(beta2), static_cast<float>(eps), static_cast<float>(wd), bc1, bc2,
                     static_cast<float>(grad_scale), inv, dt_code(g), lp_dt, cur_stream()), "adam");
}

Tensor sumsq(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "sumsq: contiguous CUDA tensor required");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = at::zeros({1}, x.options().dtype(at::kFloat));
  check_rc(oslo_sumsq(x.data_ptr(), out.data_ptr<float>(), x.numel(), dt_code(x), cur_stream()), "sumsq");
  return out;
}

Tensor ngram_ban_(const Tensor& tokens, Tensor lprobs, int64_t n) {
  TORCH_CHECK(tokens.is_cuda() && tokens.scalar_type() == at::kLong && tokens.dim() == 2 && tokens.is_contiguous(), "bad tokens");
  TORCH_CHECK(lprobs.is_cuda() && lprobs.scalar_type() == at::kFloat && lprobs.dim() == 2 && lprobs.is_contiguous() &&
                  lprobs.size(0) == tokens.size(0), "lprobs must be fp32 [rows, vocab]");
  c10::cuda::CUDAGuard guard(lprobs.device());
  check_rc(oslo_ngram_ban(reinterpret_cast<const long long*>(tokens.data_ptr<int64_t>()), lprobs.data_ptr<float>(),
                          static_cast<int>(tokens.size(0)), static_cast<int>(tokens.size(1)),
                          static_cast<int>(lprobs.size(1)), static_cast<int>(n),
                          dev_state(lprobs.get_device()).err.data_ptr<int>(), cur_stream()), "ngram_ban");
  return lprobs;
}

void check_attn_operand(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 4 && t.stride(3) == 1, name, " must be [B,H,S,D] with contiguous D");
  TORCH_CHECK(t.stride(0) % 8 == 0 && t.stride(1) % 8 == 0 && t.stride(2) % 8 == 0 &&
                  reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, " needs 16-byte aligned rows");
}

// impl 0 = mma.sync kernel (attention.cu), 1 = tcgen05/TMEM kernel (attention_sm100.cu)
std::tuple<Tensor, Tensor> flash_fwd(const Tensor& q, const Tensor& k, const Tensor& v, double scale, bool causal,
                                     int64_t window, const optional<Tensor>& kpm, int64_t impl) {
  check_attn_operand(q, "q"); check_attn_operand(k, "k"); check_attn_operand(v, "v");
  c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), H = q.size(1), Sq = q.size(2), D = q.size(3), Sk = k.size(2);
  // output laid out [B, S, H, D] in memory and returned as a [B, H, S, D] view, so merging heads is free
  Tensor o = at::empty({B, Sq, H, D}, q.options()).permute({0, 2, 1, 3});
  Tensor lse = at::empty({B, H, Sq}, q.options().dtype(at::kFloat));
  const uint8_t* mp = nullptr;
  if (kpm.has_value() && kpm->defined()) {
    TORCH_CHECK(kpm->scalar_type() == at::kByte && kpm->is_contiguous() && kpm->size(0) == B && kpm->size(1) == Sk, "bad key padding mask");
    mp = kpm->data_ptr<uint8_t>();
  }
  if (impl == 1) {
    check_rc(oslo_flash_fwd_sm100(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), mp, B, H,
                                  Sq, Sk, D, q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                  v.stride(0), v.stride(1), v.stride(2), o.stride(0), o.stride(1), o.stride(2),
                                  static_cast<float>(scale), causal ? 1 : 0, static_cast<int>(window), dt_code(q),
                                  dev_state(q.get_device()).err.data_ptr<int>(), cur_stream()), "flash_fwd_sm100");
    return {o, lse};
  }
  check_rc(oslo_flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(), mp, B, H, Sq, Sk,
                          D, q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2), v.stride(0),
                          v.stride(1), v.stride(2), o.stride(0), o.stride(1), o.stride(2), static_cast<float>(scale),
                          causal ? 1 : 0, static_cast<int>(window), dt_code(q), cur_stream()), "flash_fwd");
  return {o, lse};
}

std::tuple<Tensor, Tensor, Tensor> flash_bwd(const Tensor& dout, const Tensor& q, const Tensor& k, const Tensor& v,
                                             const Tensor& o, const Tensor& lse, double scale, bool causal,
                                             int64_t window, const optional<Tensor>& kpm, int64_t impl) {
  check_attn_operand(q, "q"); check_attn_operand(k, "k"); check_attn_operand(v, "v");
  check_attn_operand(o, "o"); check_attn_operand(dout, "dout");
  c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), H = q.size(1), Sq = q.size(2), D = q.size(3), Sk = k.size(2);
  Tensor dq = at::empty_strided(q.sizes(), q.strides(), q.options());
  Tensor dk = at::empty_strided(k.sizes(), k.strides(), k.options());
  Tensor dv = at::empty_strided(v.sizes(), v.strides(), v.options());
  Tensor delta = at::empty({B, H, Sq}, q.options().dtype(at::kFloat));
  const uint8_t* mp = (kpm.has_value() && kpm->defined()) ? kpm->data_ptr<uint8_t>() : nullptr;
  if (impl == 1) {
    check_rc(oslo_flash_bwd_sm100(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(),
                                  lse.data_ptr<float>(), delta.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(),
                                  dv.data_ptr(), mp, B, H, Sq, Sk, D, q.stride(0), q.stride(1), q.stride(2), k.stride(0),
                                  k.stride(1), k.stride(2), v.stride(0), v.stride(1), v.stride(2), o.stride(0),
                                  o.stride(1), o.stride(2), dout.stride(0), dout.stride(1), dout.stride(2),
                                  static_cast<float>(scale), causal ? 1 : 0, static_cast<int>(window), dt_code(q),
                                  dev_state(q.get_device()).err.data_ptr<int>(), cur_stream(4)), "flash_bwd_sm100");
    return {dq, dk, dv};
  }
  check_rc(oslo_flash_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), dout.data_ptr(), lse.data_ptr<float>(),
                          delta.data_ptr<float>(), nullptr, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), mp, B, H, Sq, Sk,
                          D, q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2), v.stride(0),
                          v.stride(1), v.stride(2), o.stride(0), o.stride(1), o.stride(2), dout.stride(0),
                          dout.stride(1), dout.stride(2), static_cast<float>(scale), causal ? 1 : 0,
                          static_cast<int>(window), dt_code(q), cur_stream(D > 128 ? 4 : 3)), "flash_bwd");
  return {dq, dk, dv};
}

Tensor decode_attn(const Tensor& q, const Tensor& kc, const Tensor& vc, const Tensor& lengths, double scale,
                   int64_t window) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 3 && q.is_contiguous(), "decode_attn: q must be contiguous [B,H,D]");
  TORCH_CHECK(kc.dim() == 4 && kc.is_contiguous() && vc.is_contiguous(), "decode_attn: caches must be contiguous [B,H,T,D]");
  TORCH_CHECK(lengths.scalar_type() == at::kInt && lengths.is_contiguous() && lengths.numel() == q.size(0), "bad lengths");
  c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), H = q.size(1), D = q.size(2), T = kc.size(2);
  const int sms = dev_state(q.get_device()).sms;
  int splits = std::max(1, std::min(32, (2 * sms) / std::max(1, B * H)));
  splits = std::min(splits, std::max(1, T / 32));   // at least one 8-key batch per warp and slice
  Tensor ws = at::empty({B, H, splits, D + 2}, q.options().dtype(at::kFloat));
  Tensor o = at::empty_like(q);
  check_rc(oslo_decode_attn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), lengths.data_ptr<int>(),
                            ws.data_ptr<float>(), B, H, T, D, splits, static_cast<float>(scale),
                            static_cast<int>(window), dt_code(q), dev_state(q.get_device()).err.data_ptr<int>(),
                            cur_stream(2)), "decode_attn");
  return o;
}

// GEMM fused with a collective over the symmetric buffer of a tensor-parallel group (fused_comm_gemm.cu).
// mode 1: all-reduce, the summed [M,N] is left in the staging matrix at data_off (returned view is built in
// Python); mode 2: reduce-scatter into `out` [M/world, N]; mode 3: all-gather of `a` shards, product into `out`.
int64_t gemm_comm(const Tensor& a, const Tensor& b, int64_t a_mn, int64_t b_mn, const optional<Tensor>& bias,
               const optional<Tensor>& aux, const optional<Tensor>& aux_out, const optional<Tensor>& out, int64_t flags,
               double alpha, int64_t M,
               int64_t N, int64_t K, int64_t peer_bufs_dev, int64_t own_buf, int64_t mc_base, int64_t data_off,
               int64_t flag_off, int64_t flag_bytes, int64_t rank, int64_t world, int64_t epoch, int64_t done_base,
               int64_t mode, bool use_multimem, const optional<Tensor>& trace) {
  check_2d_operand(a, "a");
  check_2d_operand(b, "b");
  TORCH_CHECK(a.scalar_type() == b.scalar_type() && (a.scalar_type() == at::kBFloat16 || a.scalar_type() == at::kHalf),
              "gemm_comm inputs must both be bf16 or fp16");
  c10::cuda::CUDAGuard guard(a.device());
  int fl = static_cast<int>(flags) & ~GEMM_FLAG_FP16;
  if (a.scalar_type() == at::kHalf) fl |= GEMM_FLAG_FP16;
  void* out_ptr = nullptr;
  int ld_out = 0;
  if (mode != 1) {
    TORCH_CHECK(out.has_value() && out->is_cuda() && out->dim() == 2 && out->stride(1) == 1 &&
                    out->scalar_type() == a.scalar_type(), "gemm_comm: bad out");
    TORCH_CHECK(out->size(1) == N && out->size(0) == (mode == 2 ? M / world : M), "gemm_comm: out shape");
    out_ptr = out->data_ptr();
    ld_out = static_cast<int>(out->stride(0));
  }
  int ld_aux_out = 0;
  if (fl & GEMM_FLAG_SAVE_PREACT) {
    TORCH_CHECK(mode == 3 && aux_out.has_value() && aux_out->size(0) == M && aux_out->size(1) == N &&
                    aux_out->stride(1) == 1, "gemm_comm: bad aux_out");
    ld_aux_out = static_cast<int>(aux_out->stride(0));
  }
  if (fl & GEMM_FLAG_BIAS) TORCH_CHECK(bias.has_value() && bias->numel() == N && bias->is_contiguous(), "bad bias");
  int ld_aux = 0;
  if (fl & GEMM_FLAG_RESIDUAL) {
    TORCH_CHECK(mode != 3 && aux.has_value() && aux->dim() == 2 && aux->size(0) == M && aux->size(1) == N &&
                    aux->stride(1) == 1 && aux->scalar_type() == a.scalar_type(), "gemm_comm: bad partial-sum operand");
    ld_aux = static_cast<int>(aux->stride(0));
  }
  auto& st = dev_state(a.get_device());
  // tile shape must be the same on every rank: decide from the problem size only
  const int wide = (N >= 256 && ((M + 127) / 128) * ((N + 255) / 256) >= usable_sms(st) / 2) ? 1 : 0;
  const int rc = oslo_gemm_comm_16bit(
      a.data_ptr(), b.data_ptr(), static_cast<int>(M), static_cast<int>(N), static_cast<int>(K),
      static_cast<int>(a.stride(0)), static_cast<int>(b.stride(0)), static_cast<int>(a_mn), static_cast<int>(b_mn),
      ptr_or_null(bias), (fl & GEMM_FLAG_RESIDUAL) ? aux->data_ptr() : nullptr, ld_aux,
      const_cast<void*>(ptr_or_null(aux_out)), ld_aux_out, fl, static_cast<float>(alpha),
      reinterpret_cast<void* const*>(peer_bufs_dev), reinterpret_cast<void*>(own_buf), reinterpret_cast<void*>(mc_base),
      data_off, flag_off, flag_bytes, static_cast<int>(rank), static_cast<int>(world), static_cast<unsigned>(epoch),
      static_cast<unsigned>(done_base), static_cast<int>(mode), use_multimem ? 1 : 0, out_ptr, ld_out, wide,
      trace.has_value() && trace->defined() ? reinterpret_cast<unsigned long long*>(trace->data_ptr<int64_t>()) : nullptr,
      st.err.data_ptr<int>(), usable_sms(st), cur_stream());
  check_rc(rc, "gemm_comm");
  // how far this call advances the slot's completion counter (the caller keeps the running total)
  const int64_t bn = wide ? 256 : 128;
  return mode == 1 ? ((M + 127) / 128) * ((N + bn - 1) / bn) * 4 : 0;
}

// In-place all-reduce of a symmetric buffer. ptr tables are device arrays of `world` addresses.
void allreduce_symm(int64_t peer_ptrs_dev, int64_t mc_ptr, int64_t signal_ptrs_dev, Tensor out, int64_t numel,
                    int64_t rank, int64_t world, bool use_multimem) {
  c10::cuda::CUDAGuard guard(out.device());
  auto& st = dev_state(out.get_device());
  check_rc(oslo_allreduce_symm(reinterpret_cast<void* const*>(peer_ptrs_dev), reinterpret_cast<void*>(mc_ptr),
                               reinterpret_cast<uint32_t* const*>(signal_ptrs_dev), out.data_ptr(), numel,
                               static_cast<int>(rank), static_cast<int>(world), dt_code(out), use_multimem ? 1 : 0,
                               st.err.data_ptr<int>(), cur_stream()), "allreduce_symm");
}

// (max, sum exp, label logit) per row combined over the ranks of a tensor-parallel group, in place
void ce_combine(Tensor mx, Tensor se, Tensor tg, int64_t peer_ptrs_dev, int64_t signal_ptrs_dev, Tensor counters,
                int64_t cap, int64_t rank, int64_t world) {
  TORCH_CHECK(mx.is_cuda() && mx.scalar_type() == at::kFloat && mx.is_contiguous() && se.is_contiguous() &&
                  tg.is_contiguous() && se.scalar_type() == at::kFloat && tg.scalar_type() == at::kFloat &&
                  se.numel() == mx.numel() && tg.numel() == mx.numel(), "ce_combine: fp32 contiguous vectors of one length");
  c10::cuda::CUDAGuard guard(mx.device());
  auto& st = dev_state(mx.get_device());
  check_rc(oslo_ce_combine(mx.data_ptr<float>(), se.data_ptr<float>(), tg.data_ptr<float>(), mx.data_ptr<float>(),
                           se.data_ptr<float>(), tg.data_ptr<float>(), reinterpret_cast<void* const*>(peer_ptrs_dev),
                           reinterpret_cast<uint32_t* const*>(signal_ptrs_dev),
                           reinterpret_cast<uint32_t*>(counters.data_ptr<int>()), static_cast<int>(mx.numel()),
                           static_cast<int>(cap), static_cast<int>(rank), static_cast<int>(world),
                           st.err.data_ptr<int>(), cur_stream()), "ce_combine");
}

// One bucket of the data-parallel gradient reduce-scatter / parameter all-gather on a symmetric flat buffer.
// `like` names the device and (reduce-scatter) the 16-bit dtype; the buffer itself is given by its address tables.
void dp_reduce_scatter(const Tensor& like, int64_t peer_ptrs_dev, int64_t mc_ptr, int64_t signal_ptrs_dev, int64_t lo,
                       int64_t hi, int64_t shard, int64_t rank, int64_t world, bool use_multimem) {
  c10::cuda::CUDAGuard guard(like.device());
  auto& st = dev_state(like.get_device());
  check_rc(oslo_dp_reduce_scatter(reinterpret_cast<void* const*>(peer_ptrs_dev), reinterpret_cast<void*>(mc_ptr),
                                  reinterpret_cast<uint32_t* const*>(signal_ptrs_dev), lo, hi, shard,
                                  static_cast<int>(rank), static_cast<int>(world), dt_code(like), use_multimem ? 1 : 0,
                                  st.err.data_ptr<int>(), cur_stream()), "dp_reduce_scatter");
}
void dp_all_gather(const Tensor& like, int64_t peer_ptrs_dev, int64_t mc_ptr, int64_t signal_ptrs_dev, int64_t lo,
                   int64_t hi, int64_t shard, int64_t rank, int64_t world, bool use_multimem) {
  c10::cuda::CUDAGuard guard(like.device());
  auto& st = dev_state(like.get_device());
  check_rc(oslo_dp_all_gather(reinterpret_cast<void* const*>(peer_ptrs_dev), reinterpret_cast<void*>(mc_ptr),
                              reinterpret_cast<uint32_t* const*>(signal_ptrs_dev), lo, hi, shard, static_cast<int>(rank),
                              static_cast<int>(world), use_multimem ? 1 : 0, st.err.data_ptr<int>(), cur_stream()),
           "dp_all_gather");
}

// y [M, N] = act([x1 | x2] @ w^T + bias) for M <= 4 rows; w [N, K1 + K2]; x1 / x2 are 2-D with contiguous last dims
Tensor gemv_rows(const Tensor& x1, const optional<Tensor>& x2, const Tensor& w, const optional<Tensor>& bias,
                 int64_t gelu_from, const optional<Tensor>& res) {
  check_2d_operand(x1, "x1");
  check_2d_operand(w, "w");
  const bool two = x2.has_value() && x2->defined();
  if (two) check_2d_operand(*x2, "x2");
  const int64_t M = x1.size(0), K1 = x1.size(1), K2 = two ? x2->size(1) : 0, N = w.size(0);
  TORCH_CHECK(w.size(1) == K1 + K2 && (!two || x2->size(0) == M), "gemv_rows: shapes do not match");
  TORCH_CHECK(x1.scalar_type() == w.scalar_type() && (!two || x2->scalar_type() == w.scalar_type()), "gemv_rows: dtypes differ");
  const bool has_bias = bias.has_value() && bias->defined();
  if (has_bias) TORCH_CHECK(bias->numel() == N && bias->scalar_type() == w.scalar_type() && bias->is_contiguous(), "bad bias");
  const bool has_res = res.has_value() && res->defined();
  if (has_res)
    TORCH_CHECK(res->dim() == 2 && res->size(0) == M && res->size(1) == N && res->stride(1) == 1 &&
                    res->scalar_type() == w.scalar_type(), "bad residual");
  c10::cuda::CUDAGuard guard(x1.device());
  Tensor y = at::empty({M, N}, x1.options());
  auto& st = dev_state(x1.get_device());
  check_rc(oslo_gemv_rows(x1.data_ptr(), static_cast<int>(x1.stride(0)), static_cast<int>(K1),
                          two ? x2->data_ptr() : nullptr, two ? static_cast<int>(x2->stride(0)) : 0, static_cast<int>(K2),
                          w.data_ptr(), static_cast<int>(w.stride(0)), has_bias ? bias->data_ptr() : nullptr,
                          has_res ? res->data_ptr() : nullptr, has_res ? static_cast<int>(res->stride(0)) : 0, y.data_ptr(),
                          static_cast<int>(N), static_cast<int>(M), static_cast<int>(N), static_cast<int>(gelu_from),
                          dt_code(x1), usable_sms(st), cur_stream()), "gemv_rows");
  return y;
}

// GPT-J rotary on q, k ([B, H*D] row slices) + append of k, v to the static cache at the device-side position
Tensor rotary_append(const Tensor& q, const Tensor& k, const Tensor& v, Tensor kc, Tensor vc, const Tensor& lengths,
                     const Tensor& write_index, int64_t rotary_dim, double base) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 2 && k.dim() == 2 && v.dim() == 2 && q.stride(1) == 1 && k.stride(1) == 1 &&
                  v.stride(1) == 1, "rotary_append: q, k, v must be [B, H*D] with contiguous last dim");
  TORCH_CHECK(kc.dim() == 4 && kc.is_contiguous() && vc.is_contiguous() && kc.sizes() == vc.sizes(), "bad cache");
  TORCH_CHECK(lengths.scalar_type() == at::kInt && write_index.scalar_type() == at::kLong, "bad position tensors");
  const int64_t B = kc.size(0), H = kc.size(1), T = kc.size(2), D = kc.size(3);
  TORCH_CHECK(q.size(0) == B && q.size(1) == H * D && k.size(1) == H * D && v.size(1) == H * D, "shape mismatch");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor q_out = at::empty({B, H, D}, q.options());
  check_rc(oslo_rotary_append(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0),
                              q_out.data_ptr(), kc.data_ptr(), vc.data_ptr(), lengths.data_ptr<int>(),
                              reinterpret_cast<const long long*>(write_index.data_ptr<int64_t>()), static_cast<int>(B),
                              static_cast<int>(H), static_cast<int>(D), static_cast<int>(T), static_cast<int>(rotary_dim),
                              static_cast<float>(base), dt_code(q), dev_state(q.get_device()).err.data_ptr<int>(),
                              cur_stream()), "rotary_append");
  return q_out;
}

// Vocab-parallel embedding: ids int64 [tokens], weight = this rank's [hi - lo, H] shard; returns [tokens, H]
Tensor vocab_embed(const Tensor& ids, const Tensor& weight, int64_t lo, int64_t hi, int64_t peer_ptrs_dev,
                   int64_t mc_ptr, int64_t signal_ptrs_dev, Tensor counters, int64_t half_bytes, int64_t rank,
                   int64_t world, bool use_multimem) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous(), "vocab_embed: ids must be contiguous int64");
  TORCH_CHECK(weight.is_cuda() && weight.dim() == 2 && weight.is_contiguous() && weight.size(0) == hi - lo, "vocab_embed: bad weight shard");
  TORCH_CHECK(counters.is_cuda() && counters.scalar_type() == at::kInt && counters.numel() >= 64, "vocab_embed: bad counters");
  c10::cuda::CUDAGuard guard(ids.device());
  const int64_t tokens = ids.numel(), H = weight.size(1);
  Tensor out = at::empty({tokens, H}, weight.options());
  auto& st = dev_state(ids.get_device());
  check_rc(oslo_vocab_embed(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), weight.data_ptr(), out.data_ptr(),
                            reinterpret_cast<void* const*>(peer_ptrs_dev), reinterpret_cast<void*>(mc_ptr),
                            reinterpret_cast<uint32_t* const*>(signal_ptrs_dev),
                            reinterpret_cast<uint32_t*>(counters.data_ptr<int>()), tokens, static_cast<int>(H), lo, hi,
                            half_bytes, static_cast<int>(rank), static_cast<int>(world), dt_code(weight),
                            use_multimem ? 1 : 0, st.err.data_ptr<int>(), usable_sms(st), cur_stream()), "vocab_embed");
  return out;
}

// Wait (bounded by limit_ms, at most 1000) until flag[0] >= target; returns the nanoseconds spent. A wait that runs
// out leaves ERR_WAIT_PEER in the device error word, exactly like the waits inside the communication kernels.
Tensor wait_probe(const Tensor& flag, int64_t target, double limit_ms) {
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == at::kInt && flag.numel() >= 1, "wait_probe: int32 CUDA flag");
  c10::cuda::CUDAGuard guard(flag.device());
  Tensor waited = at::zeros({1}, flag.options().dtype(at::kLong));
  auto& st = dev_state(flag.get_device());
  check_rc(oslo_wait_probe(reinterpret_cast<const uint32_t*>(flag.data_ptr<int>()), static_cast<uint32_t>(target),
                           static_cast<unsigned long long>(limit_ms * 1e6), st.err.data_ptr<int>(),
                           reinterpret_cast<unsigned long long*>(waited.data_ptr<int64_t>()), cur_stream()), "wait_probe");
  return waited;
}

// In-place one-kernel all-reduce of a small tensor through two alternating staging halves of a symmetric buffer.
void allreduce_oneshot(Tensor x, int64_t peer_ptrs_dev, int64_t mc_ptr, int64_t signal_ptrs_dev, Tensor counters,
                       int64_t stage_off, int64_t half_bytes, int64_t rank, int64_t world, bool use_multimem) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && counters.is_cuda() && counters.scalar_type() == at::kInt &&
                  counters.numel() >= 64, "allreduce_oneshot: bad arguments");
  c10::cuda::CUDAGuard guard(x.device());
  auto& st = dev_state(x.get_device());
  check_rc(oslo_allreduce_oneshot(x.data_ptr(), x.data_ptr(), reinterpret_cast<void* const*>(peer_ptrs_dev),
                                  reinterpret_cast<void*>(mc_ptr), reinterpret_cast<uint32_t* const*>(signal_ptrs_dev),
                                  reinterpret_cast<uint32_t*>(counters.data_ptr<int>()), x.numel(), stage_off, half_bytes,
                                  static_cast<int>(rank), static_cast<int>(world), dt_code(x), use_multimem ? 1 : 0,
                                  st.err.data_ptr<int>(), cur_stream()), "allreduce_oneshot");
}

}  // namespace

// Schemas. Kernels that take tensors are registered for the CUDA dispatch key (below), which leaves the Meta /
// fake-tensor slot free for the shape implementations that oslo_b200/ops/fake_impls.py registers from Python.
TORCH_LIBRARY(oslo_b200, m) {
  m.def("error_word(Tensor like) -> Tensor");
  m.def("launch_count() -> int", &launch_count);
  m.def("set_reserved_sms(int n) -> int", &set_reserved_sms);
  m.def("reserved_sms() -> int", &reserved_sms);
  m.def("gemm(Tensor a, Tensor b, int a_mn, int b_mn, Tensor? bias, Tensor? aux, Tensor(a!)? out, Tensor(b!)? aux_out, int flags, float alpha) -> Tensor");
  m.def("gemm_ce_stats(Tensor a, Tensor b, int b_mn, Tensor? bias, Tensor labels, int vocab_start) -> (Tensor, Tensor, Tensor)");
  m.def("gemm_ce_grad(Tensor a, Tensor b, int b_mn, Tensor? bias, Tensor labels, int vocab_start, Tensor lse, Tensor scale) -> Tensor");
  m.def("gemm_small_m(Tensor a, Tensor b, int b_mn, Tensor? bias, int gelu_from) -> Tensor");
  m.def("layernorm_fwd(Tensor x, Tensor w, Tensor? b, float eps) -> (Tensor, Tensor, Tensor)");
  m.def("layernorm_bwd(Tensor dy, Tensor x, Tensor w, Tensor mean, Tensor rstd) -> (Tensor, Tensor, Tensor)");
  m.def("bias_gelu_fwd(Tensor x, Tensor? bias) -> Tensor");
  m.def("bias_gelu_bwd(Tensor dy, Tensor x, Tensor? bias) -> Tensor");
  m.def("bias_dropout_residual(Tensor x, Tensor? bias, Tensor? residual, float p, int seed, int mode) -> Tensor");
  m.def("colsum(Tensor x) -> Tensor");
  m.def("rotary(Tensor x, Tensor positions, int rotary_dim, float base, bool inverse) -> Tensor");
  m.def("rotary_(Tensor(a!) x, Tensor positions, int heads, int head_dim, int rotary_dim, float base, bool inverse) -> Tensor(a!)");
  m.def("causal_softmax_fwd(Tensor x, float scale) -> Tensor");
  m.def("masked_softmax_fwd(Tensor x, Tensor mask, float scale) -> Tensor");
  m.def("softmax_bwd(Tensor y, Tensor dy, float scale) -> Tensor");
  m.def("ce_stats(Tensor logits, Tensor labels, int vocab_start) -> (Tensor, Tensor, Tensor)");
  m.def("ce_grad_(Tensor(a!) logits, Tensor labels, int vocab_start, Tensor lse, Tensor scale) -> Tensor(a!)");
  m.def("adam_step(Tensor(a!) p, Tensor g, Tensor(b!) m, Tensor(c!) v, Tensor(d!)? p_lp, float lr, float beta1, float beta2, float eps, float wd, int step, float grad_scale, Tensor? inv_scale) -> ()");
  m.def("sumsq(Tensor x) -> Tensor");
  m.def("ngram_ban_(Tensor tokens, Tensor(a!) lprobs, int n) -> Tensor(a!)");
  m.def("flash_fwd(Tensor q, Tensor k, Tensor v, float scale, bool causal, int window, Tensor? kpm, int impl=1) -> (Tensor, Tensor)");
  m.def("flash_bwd(Tensor dout, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse, float scale, bool causal, int window, Tensor? kpm, int impl=1) -> (Tensor, Tensor, Tensor)");
  m.def("decode_attn(Tensor q, Tensor kc, Tensor vc, Tensor lengths, float scale, int window) -> Tensor");
  m.def("gemm_comm(Tensor a, Tensor b, int a_mn, int b_mn, Tensor? bias, Tensor? aux, Tensor(a!)? aux_out, Tensor(b!)? out, int flags, float alpha, int M, int N, int K, int peer_bufs_dev, int own_buf, int mc_base, int data_off, int flag_off, int flag_bytes, int rank, int world, int epoch, int done_base, int mode, bool use_multimem, Tensor(c!)? trace) -> int");
  m.def("gemv_rows(Tensor x1, Tensor? x2, Tensor w, Tensor? bias, int gelu_from, Tensor? res=None) -> Tensor");
  m.def("rotary_append(Tensor q, Tensor k, Tensor v, Tensor(a!) kc, Tensor(b!) vc, Tensor lengths, Tensor write_index, int rotary_dim, float base) -> Tensor");
  m.def("vocab_embed(Tensor ids, Tensor weight, int lo, int hi, int peer_ptrs_dev, int mc_ptr, int signal_ptrs_dev, Tensor(a!) counters, int half_bytes, int rank, int world, bool use_multimem) -> Tensor");
  m.def("wait_probe(Tensor flag, int target, float limit_ms) -> Tensor");
  m.def("allreduce_oneshot(Tensor(a!) x, int peer_ptrs_dev, int mc_ptr, int signal_ptrs_dev, Tensor(b!) counters, int stage_off, int half_bytes, int rank, int world, bool use_multimem) -> ()");
  m.def("ce_combine(Tensor(a!) mx, Tensor(b!) se, Tensor(c!) tg, int peer_ptrs_dev, int signal_ptrs_dev, Tensor(d!) counters, int cap, int rank, int world) -> ()");
  m.def("dp_reduce_scatter(Tensor like, int peer_ptrs_dev, int mc_ptr, int signal_ptrs_dev, int lo, int hi, int shard, int rank, int world, bool use_multimem) -> ()");
  m.def("dp_all_gather(Tensor like, int peer_ptrs_dev, int mc_ptr, int signal_ptrs_dev, int lo, int hi, int shard, int rank, int world, bool use_multimem) -> ()");
  m.def("allreduce_symm(int peer_ptrs_dev, int mc_ptr, int signal_ptrs_dev, Tensor(a!) out, int numel, int rank, int world, bool use_multimem) -> ()");
}

TORCH_LIBRARY_IMPL(oslo_b200, CUDA, m) {
  m.impl("error_word", &error_word);
  m.impl("gemm", &gemm);
  m.impl("gemm_small_m", &gemm_small_m);
  m.impl("gemm_ce_stats", &gemm_ce_stats);
  m.impl("gemm_ce_grad", &gemm_ce_grad);
  m.impl("layernorm_fwd", &layernorm_fwd);
  m.impl("layernorm_bwd", &layernorm_bwd);
  m.impl("bias_gelu_fwd", &bias_gelu_fwd);
  m.impl("bias_gelu_bwd", &bias_gelu_bwd);
  m.impl("bias_dropout_residual", &bias_dropout_residual);
  m.impl("colsum", &colsum);
  m.impl("rotary", &rotary);
  m.impl("rotary_", &rotary_);
  m.impl("causal_softmax_fwd", &causal_softmax_fwd);
  m.impl("masked_softmax_fwd", &masked_softmax_fwd);
  m.impl("softmax_bwd", &softmax_bwd);
  m.impl("ce_stats", &ce_stats);
  m.impl("ce_grad_", &ce_grad_);
  m.impl("adam_step", &adam_step);
  m.impl("sumsq", &sumsq);
  m.impl("ngram_ban_", &ngram_ban_);
  m.impl("flash_fwd", &flash_fwd);
  m.impl("flash_bwd", &flash_bwd);
  m.impl("decode_attn", &decode_attn);
  m.impl("gemm_comm", &gemm_comm);
  m.impl("gemv_rows", &gemv_rows);
  m.impl("rotary_append", &rotary_append);
  m.impl("vocab_embed", &vocab_embed);
  m.impl("wait_probe", &wait_probe);
  m.impl("allreduce_oneshot", &allreduce_oneshot);
  m.impl("allreduce_symm", &allreduce_symm);
  m.impl("ce_combine", &ce_combine);
  m.impl("dp_reduce_scatter", &dp_reduce_scatter);
  m.impl("dp_all_gather", &dp_all_gather);
}
