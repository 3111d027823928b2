// Python module _flagcx_torch: the c10d backend and the fused training ops.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/chrono.h>
#include <torch/extension.h>

#include "train_ops.h"

namespace fcxt {
void bindBackend(py::module &m);
void bindFused(py::module &m);  // fused_ops.cpp

#define CUDA_OK(call)                                                                     \
  do {                                                                                    \
    cudaError_t _e = (call);                                                              \
    TORCH_CHECK(_e == cudaSuccess, "flagcx op failed: ", cudaGetErrorString(_e), " in ", #call); \
  } while (0)

static void checkBf16(const at::Tensor &t, const char *name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), name, " must be a contiguous bf16 CUDA tensor");
}

static cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }

// (residual_out, y, mean, rstd) = LN(x + delta).  With delta undefined, residual_out is x itself.
static std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> layernormFwd(const at::Tensor &x, const c10::optional<at::Tensor> &delta,
                                                                              const at::Tensor &gamma, const at::Tensor &beta, double eps) {
  checkBf16(x, "x");
  checkBf16(gamma, "gamma");
  checkBf16(beta, "beta");
  c10::cuda::CUDAGuard g(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  at::Tensor res = x;
  const void *dptr = nullptr;
  if (delta.has_value() && delta->defined()) {
    checkBf16(*delta, "delta");
    res = at::empty_like(x);
    dptr = delta->data_ptr();
  }
  auto y = at::empty_like(x);
  auto stats = at::empty({2, M}, x.options().dtype(at::kFloat));
  CUDA_OK(fcxLayerNormFwd(x.data_ptr(), dptr, gamma.data_ptr(), beta.data_ptr(), dptr ? res.data_ptr() : nullptr, y.data_ptr(),
                          stats.data_ptr<float>(), stats.data_ptr<float>() + M, M, C, (float)eps, cur()));
  return {res, y, stats[0], stats[1]};
}

// dx (+ dres), dgamma, dbeta
static std::tuple<at::Tensor, at::Tensor, at::Tensor> layernormBwd(const at::Tensor &dy, const at::Tensor &x, const at::Tensor &gamma,
                                                                  const at::Tensor &mean, const at::Tensor &rstd,
                                                                  const c10::optional<at::Tensor> &dres) {
  checkBf16(dy, "dy");
  checkBf16(x, "x");
  c10::cuda::CUDAGuard g(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  auto dx = at::empty_like(x);
  auto dgamma = at::empty_like(gamma), dbeta = at::empty_like(gamma);
  auto partial = at::empty({fcxLnPartials(M), 2, C}, x.options().dtype(at::kFloat));
  const void *dr = dres.has_value() && dres->defined() ? dres->data_ptr() : nullptr;
  CUDA_OK(fcxLayerNormBwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), dr,
                          dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), partial.data_ptr<float>(), M, C, 0, cur()));
  return {dx, dgamma, dbeta};
}

static at::Tensor biasGeluFwd(const at::Tensor &x, const at::Tensor &bias) {
  checkBf16(x, "x");
  checkBf16(bias, "bias");
  c10::cuda::CUDAGuard g(x.device());
  const int C = (int)x.size(-1);
  auto y = at::empty_like(x);
  CUDA_OK(fcxBiasGeluFwd(x.data_ptr(), bias.data_ptr(), y.data_ptr(), x.numel() / C, C, cur()));
  return y;
}

// returns (dx, dbias)
static std::tuple<at::Tensor, at::Tensor> biasGeluBwd(const at::Tensor &dy, const at::Tensor &x, const at::Tensor &bias) {
  checkBf16(dy, "dy");
  checkBf16(x, "x");
  c10::cuda::CUDAGuard g(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  auto dx = at::empty_like(x);
  CUDA_OK(fcxBiasGeluBwd(dy.data_ptr(), x.data_ptr(), bias.data_ptr(), dx.data_ptr(), M, C, cur()));
  auto dbias = at::empty_like(bias);
  auto partial = at::empty({fcxColSumPartials(M), C}, x.options().dtype(at::kFloat));
  CUDA_OK(fcxColSum(dx.data_ptr(), dbias.data_ptr(), partial.data_ptr<float>(), M, C, 0, cur()));
  return {dx, dbias};
}

static at::Tensor colSum(const at::Tensor &a) {
  checkBf16(a, "a");
  c10::cuda::CUDAGuard g(a.device());
  const int C = (int)a.size(-1), M = (int)(a.numel() / C);
  auto out = at::empty({C}, a.options());
  auto partial = at::empty({fcxColSumPartials(M), C}, a.options().dtype(at::kFloat));
  CUDA_OK(fcxColSum(a.data_ptr(), out.data_ptr(), partial.data_ptr<float>(), M, C, 0, cur()));
  return out;
}

// In place: logits become d(mean loss)/d(logits) * grad_scale; returns per-row losses (fp32).
static at::Tensor crossEntropy(at::Tensor &logits, const at::Tensor &targets, int64_t vocab, double gradScale) {
  checkBf16(logits, "logits");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous(), "targets must be int64 CUDA");
  c10::cuda::CUDAGuard g(logits.device());
  const int Vpad = (int)logits.size(-1), M = (int)(logits.numel() / Vpad);
  TORCH_CHECK(targets.numel() == M, "one target per row");
  auto losses = at::empty({M}, logits.options().dtype(at::kFloat));
  CUDA_OK(fcxCrossEntropyFwdBwd(logits.data_ptr(), targets.data_ptr<int64_t>(), losses.data_ptr<float>(), M, (int)vocab, Vpad,
                                (float)gradScale, cur()));
  return losses;
}

static void adamw(at::Tensor &master, at::Tensor &param, at::Tensor &grad, at::Tensor &m, at::Tensor &v, double lr, double b1, double b2,
                  double eps, double wd, int64_t step, double gradScale, bool zeroGrad) {
  TORCH_CHECK(master.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat, "fp32 state");
  checkBf16(param, "param");
  checkBf16(grad, "grad");
  c10::cuda::CUDAGuard g(master.device());
  size_t n = master.numel();
  TORCH_CHECK((size_t)param.numel() == n && (size_t)grad.numel() == n && (size_t)m.numel() == n && (size_t)v.numel() == n, "size mismatch");
  CUDA_OK(fcxAdamW(master.data_ptr<float>(), param.data_ptr(), grad.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(), n, (float)lr,
                   (float)b1, (float)b2, (float)eps, (float)wd, (int)step, (float)gradScale, zeroGrad ? 1 : 0, cur()));
}

}  // namespace fcxt

PYBIND11_MODULE(_flagcx_torch, m) {
  m.doc() = "flagcx_b200 native PyTorch pieces: c10d backend 'flagcx' and fused sm_100a ops";
  fcxt::bindBackend(m);
  fcxt::bindFused(m);
  m.def("layernorm_fwd", &fcxt::layernormFwd, py::arg("x"), py::arg("delta"), py::arg("gamma"), py::arg("beta"), py::arg("eps") = 1e-5);
  m.def("layernorm_bwd", &fcxt::layernormBwd);
  m.def("bias_gelu_fwd", &fcxt::biasGeluFwd);
  m.def("bias_gelu_bwd", &fcxt::biasGeluBwd);
  m.def("col_sum", &fcxt::colSum);
  m.def("cross_entropy_", &fcxt::crossEntropy);
  m.def("adamw_", &fcxt::adamw);
}
