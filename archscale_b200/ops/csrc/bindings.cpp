// Python bindings: torch tensors in, raw pointers to the C entry points of api.h out.
// Output tensors are allocated here with torch's caching allocator on the current stream.
#include <cstdlib>
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "api.h"

namespace {

inline int dcode(const at::Tensor& t) {
  if (t.scalar_type() == at::kFloat) return 0;
  if (t.scalar_type() == at::kBFloat16) return 1;
  TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
}
inline int dcode_opt(const c10::optional<at::Tensor>& t, int dflt) { return t.has_value() ? dcode(*t) : dflt; }
inline const void* ptr_opt(const c10::optional<at::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }
inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void check(int rc, const char* what) { TORCH_CHECK(rc == 0, what, " failed with code ", rc); }

int g_num_sms = 0;
at::Tensor g_status;  // int32 [1] per process: device-side error word of the tcgen05 kernels

int num_sms() {
  if (!g_num_sms) g_num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return g_num_sms;
}
at::Tensor g_splitk_sem;  // counters of the serial split-K weight-gradient path (see gemm_bf16.cu)
void ensure_splitk_workspace(const at::Device& dev) {
  if (!g_splitk_sem.defined()) {
    g_splitk_sem = at::zeros({1 << 16}, at::TensorOptions().dtype(at::kInt).device(dev));
    b200_gemm_set_splitk_workspace(reinterpret_cast<uint32_t*>(g_splitk_sem.data_ptr<int>()), 1 << 16);
  }
}
int* status_ptr(const at::Device& dev) {
  if (!g_status.defined()) g_status = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(dev));
  return g_status.data_ptr<int>();
}

// ---- GEMM ---------------------------------------------------------------------------------
// ARCHSCALE_B200_GEMM=1cta forces the one-CTA 128×256 kernel; otherwise plain GEMMs pair two SMs on a 256×256 tile.
static int g_gemm_pair = -1;
static bool gemm_use_pair() {
  if (g_gemm_pair < 0) { const char* v = std::getenv("ARCHSCALE_B200_GEMM"); g_gemm_pair = (v != nullptr && std::string(v) == "1cta") ? 0 : 1; }
  return g_gemm_pair == 1;
}
// tests switch between the two kernels at run time; returns the previous setting
static bool set_gemm_pair(bool on) { const bool was = gemm_use_pair(); g_gemm_pair = on ? 1 : 0; return was; }
// mode 0: a[M,K] b[N,K] ; 1: a[M,K] b[K,N] ; 2: a[K,M] b[K,N].  `acc`: fp32 [M,N] accumulated in place.
at::Tensor gemm_bf16(const at::Tensor& a, const at::Tensor& b, int64_t mode, at::ScalarType out_dtype,
                     const c10::optional<at::Tensor>& acc) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1);
  c10::cuda::CUDAGuard guard(a.device());
  int64_t M, N, K;
  if (mode == 0) { M = a.size(0); K = a.size(1); N = b.size(0); TORCH_CHECK(b.size(1) == K); }
  else if (mode == 1) { M = a.size(0); K = a.size(1); N = b.size(1); TORCH_CHECK(b.size(0) == K); }
  else { K = a.size(0); M = a.size(1); N = b.size(1); TORCH_CHECK(b.size(0) == K); }
  at::Tensor out;
  int accumulate = 0;
  if (acc.has_value()) {
    out = *acc;
    TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous() && out.size(0) == M && out.size(1) == N);
    accumulate = 1;
  } else {
    out = at::empty({M, N}, a.options().dtype(out_dtype));
  }
  const int out_f32 = out.scalar_type() == at::kFloat;
  // accumulating (weight-gradient) GEMMs may split K; the counters are shared, so such GEMMs must not overlap on
  // different streams (they are all issued on the autograd stream).  ARCHSCALE_B200_NO_SPLITK=1 turns it off.
  static const bool no_splitk = std::getenv("ARCHSCALE_B200_NO_SPLITK") != nullptr;
  if (accumulate && !no_splitk) ensure_splitk_workspace(a.device());
  if (gemm_use_pair()) {
    check(b200_gemm2_bf16((int)mode, a.data_ptr(), b.data_ptr(), out.data_ptr(), nullptr, (int)M, (int)N, (int)K,
                          (int)a.stride(0), (int)b.stride(0), (int)out.stride(0), 1.f, 0.f, out_f32, accumulate, num_sms(),
                          status_ptr(a.device()), cur_stream()), "gemm2_bf16");
    return out;
  }
  check(b200_gemm_bf16((int)mode, a.data_ptr(), b.data_ptr(), out.data_ptr(), nullptr, (int)M, (int)N, (int)K,
                       (int)a.stride(0), (int)b.stride(0), (int)out.stride(0), 1.f, 0.f, out_f32, accumulate, num_sms(),
                       status_ptr(a.device()), cur_stream()), "gemm_bf16");
  return out;
}

// out(bf16) = alpha · op(a)·op(b) + beta · c
at::Tensor gemm_bf16_epi(const at::Tensor& a, const at::Tensor& b, int64_t mode, double alpha, double beta,
                         const c10::optional<at::Tensor>& c) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(a.device());
  int64_t M, N, K;
  if (mode == 0) { M = a.size(0); K = a.size(1); N = b.size(0); }
  else if (mode == 1) { M = a.size(0); K = a.size(1); N = b.size(1); }
  else { K = a.size(0); M = a.size(1); N = b.size(1); }
  at::Tensor out = at::empty({M, N}, a.options());
  if (c.has_value()) TORCH_CHECK(c->is_contiguous() && c->scalar_type() == at::kBFloat16 && c->size(0) == M && c->size(1) == N);
  check((gemm_use_pair() ? b200_gemm2_bf16 : b200_gemm_bf16)((int)mode, a.data_ptr(), b.data_ptr(), out.data_ptr(), ptr_opt(c), (int)M, (int)N,
                       (int)K, (int)a.stride(0), (int)b.stride(0), (int)N, (float)alpha, (float)beta, 0, 0, num_sms(),
                       status_ptr(a.device()), cur_stream()), "gemm_bf16_epi");
  return out;
}

int64_t device_status() {
  if (!g_status.defined()) return 0;
  return g_status.item<int>();
}
void reset_device_status() { if (g_status.defined()) g_status.zero_(); }

// ---- RMSNorm ------------------------------------------------------------------------------
std::tuple<at::Tensor, at::Tensor> rmsnorm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& w, double eps,
                                               c10::optional<at::ScalarType> out_dtype) {
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), cols = x.size(1);
  at::Tensor out = at::empty({rows, cols}, x.options().dtype(out_dtype.value_or(x.scalar_type())));
  at::Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  check(b200_rmsnorm_fwd(x.data_ptr(), dcode(x), ptr_opt(w), dcode_opt(w, 0), out.data_ptr(), dcode(out),
                         rstd.data_ptr<float>(), (int)rows, (int)cols, (float)eps, cur_stream()), "rmsnorm_fwd");
  return {out, rstd};
}

std::tuple<at::Tensor, at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const c10::optional<at::Tensor>& w,
                                               const at::Tensor& rstd) {
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), cols = x.size(1);
  at::Tensor dx = at::empty_like(x);
  at::Tensor dw, part;
  if (w.has_value()) {
    dw = at::empty({cols}, x.options().dtype(at::kFloat));
    part = at::empty({b200_rmsnorm_bwd_partials((int)rows, (int)cols), cols}, x.options().dtype(at::kFloat));
  }
  check(b200_rmsnorm_bwd(dy.data_ptr(), dcode(dy), x.data_ptr(), dcode(x), ptr_opt(w), dcode_opt(w, 0),
                         rstd.data_ptr<float>(), dx.data_ptr(), w.has_value() ? part.data_ptr<float>() : nullptr,
                         w.has_value() ? dw.data_ptr<float>() : nullptr, (int)rows, (int)cols, cur_stream()), "rmsnorm_bwd");
  return {dx, dw};
}

// ---- SwiGLU -------------------------------------------------------------------------------
at::Tensor swiglu_fwd(const at::Tensor& g, const at::Tensor& u) {
  c10::cuda::CUDAGuard guard(g.device());
  at::Tensor y = at::empty_like(g);
  check(b200_swiglu_fwd(g.data_ptr(), u.data_ptr(), y.data_ptr(), g.numel(), cur_stream()), "swiglu_fwd");
  return y;
}
std::tuple<at::Tensor, at::Tensor> swiglu_bwd(const at::Tensor& g, const at::Tensor& u, const at::Tensor& dy) {
  c10::cuda::CUDAGuard guard(g.device());
  at::Tensor dg = at::empty_like(g), du = at::empty_like(u);
  check(b200_swiglu_bwd(g.data_ptr(), u.data_ptr(), dy.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(), cur_stream()), "swiglu_bwd");
  return {dg, du};
}
at::Tensor swiglu_packed_fwd(const at::Tensor& x) {
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), I = x.size(1) / 2;
  at::Tensor y = at::empty({rows, I}, x.options());
  check(b200_swiglu_packed_fwd(x.data_ptr(), y.data_ptr(), rows, (int)I, cur_stream()), "swiglu_packed_fwd");
  return y;
}
at::Tensor swiglu_packed_bwd(const at::Tensor& x, const at::Tensor& dy) {
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), I = x.size(1) / 2;
  at::Tensor dx = at::empty_like(x);
  check(b200_swiglu_packed_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), rows, (int)I, cur_stream()), "swiglu_packed_bwd");
  return dx;
}

// ---- cross entropy -------------------------------------------------------------------------
at::Tensor cross_entropy_fwd_bwd_(at::Tensor& logits, const at::Tensor& target, int64_t ignore_index, double ls, double zs) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && target.scalar_type() == at::kLong && target.is_contiguous());
  at::Tensor loss = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  check(b200_cross_entropy_fwd_bwd(logits.data_ptr(), dcode(logits), target.data_ptr<int64_t>(), loss.data_ptr<float>(),
                                   (int)logits.size(0), (int)logits.size(1), logits.stride(0), (int)ignore_index, (float)ls,
                                   (float)zs, cur_stream()), "cross_entropy_fwd_bwd");
  return loss;
}

// ---- QK-norm + RoPE --------------------------------------------------------------------------
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> qknorm_rope_fwd(
    const at::Tensor& q, const at::Tensor& k, const c10::optional<at::Tensor>& qw, const c10::optional<at::Tensor>& kw,
    const c10::optional<at::Tensor>& cos, const c10::optional<at::Tensor>& sin, double eps) {
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), T = q.size(1), H = q.size(2), D = q.size(3), G = k.size(2);
  // q / k may be column slices of a wider matrix: rows of heads must be dense, tokens a uniform stride apart
  auto tok_stride = [](const at::Tensor& t) {
    TORCH_CHECK(t.stride(3) == 1 && t.stride(2) == t.size(3) && (t.size(0) == 1 || t.stride(0) == t.size(1) * t.stride(1)),
                "qknorm_rope: unsupported strides");
    return t.stride(1);
  };
  const int64_t q_ts = tok_stride(q), k_ts = tok_stride(k);
  at::Tensor qo = at::empty({B, T, H, D}, q.options()), ko = at::empty({B, T, G, D}, k.options()), qr, kr;
  if (qw.has_value()) {
    qr = at::empty({B * T * H}, q.options().dtype(at::kFloat));
    kr = at::empty({B * T * G}, q.options().dtype(at::kFloat));
  }
  check(b200_qknorm_rope_fwd(q.data_ptr(), k.data_ptr(), ptr_opt(qw), ptr_opt(kw), dcode_opt(qw, 0), ptr_opt(cos),
                             ptr_opt(sin), qo.data_ptr(), ko.data_ptr(), qw.has_value() ? qr.data_ptr<float>() : nullptr,
                             qw.has_value() ? kr.data_ptr<float>() : nullptr, B * T, (int)T, (int)H, (int)G, (int)D,
                             (float)eps, q_ts, k_ts, cur_stream()), "qknorm_rope_fwd");
  return {qo, ko, qr, kr};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> qknorm_rope_bwd(
    const at::Tensor& dqo, const at::Tensor& dko, const at::Tensor& q, const at::Tensor& k,
    const c10::optional<at::Tensor>& qw, const c10::optional<at::Tensor>& kw, const c10::optional<at::Tensor>& cos,
    const c10::optional<at::Tensor>& sin, const c10::optional<at::Tensor>& q_rstd, const c10::optional<at::Tensor>& k_rstd) {
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), T = q.size(1), H = q.size(2), D = q.size(3), G = k.size(2);
  TORCH_CHECK(dqo.is_contiguous() && dko.is_contiguous());
  at::Tensor dq = at::empty({B, T, H, D}, q.options()), dk = at::empty({B, T, G, D}, k.options()), dqw, dkw, part;
  if (qw.has_value()) {
    dqw = at::empty({D}, q.options().dtype(at::kFloat));
    dkw = at::empty({D}, q.options().dtype(at::kFloat));
    part = at::empty({b200_qknorm_rope_grid(), 2, D}, q.options().dtype(at::kFloat));
  }
  check(b200_qknorm_rope_bwd(dqo.data_ptr(), dko.data_ptr(), q.data_ptr(), k.data_ptr(), ptr_opt(qw), ptr_opt(kw),
                             dcode_opt(qw, 0), ptr_opt(cos), ptr_opt(sin),
                             q_rstd.has_value() ? q_rstd->data_ptr<float>() : nullptr,
                             k_rstd.has_value() ? k_rstd->data_ptr<float>() : nullptr, dq.data_ptr(), dk.data_ptr(),
                             qw.has_value() ? dqw.data_ptr<float>() : nullptr, qw.has_value() ? dkw.data_ptr<float>() : nullptr,
                             qw.has_value() ? part.data_ptr<float>() : nullptr, B * T, (int)T, (int)H, (int)G, (int)D,
                             q.stride(1), k.stride(1), cur_stream()), "qknorm_rope_bwd");
  return {dq, dk, dqw, dkw};
}

}  // namespace

#include "bindings_extra.inc"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm_bf16", &gemm_bf16, "bf16 tcgen05 GEMM", py::arg("a"), py::arg("b"), py::arg("mode"), py::arg("out_dtype"),
        py::arg("acc") = py::none());
  m.def("gemm_bf16_epi", &gemm_bf16_epi);
  m.def("set_gemm_pair", &set_gemm_pair);
  m.def("gemm_pair", &gemm_use_pair);
  m.def("device_status", &device_status);
  m.def("reset_device_status", &reset_device_status);
  m.def("rmsnorm_fwd", &rmsnorm_fwd, py::arg("x"), py::arg("w"), py::arg("eps"), py::arg("out_dtype") = py::none());
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("swiglu_packed_fwd", &swiglu_packed_fwd);
  m.def("swiglu_packed_bwd", &swiglu_packed_bwd);
  m.def("cross_entropy_fwd_bwd_", &cross_entropy_fwd_bwd_);
  m.def("qknorm_rope_fwd", &qknorm_rope_fwd);
  m.def("qknorm_rope_bwd", &qknorm_rope_bwd);
  register_extra(m);
}
