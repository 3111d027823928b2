// Python module _flagcx_torch: the c10d backend and the fused training ops.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/chrono.h>
#include <torch/extension.h>

#include "flagcx.h"
#include "flagcx_ext.h"
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
                                                                  const c10::optional<at::Tensor> &dres,
                                                                  const c10::optional<at::Tensor> &dgammaInto,
                                                                  const c10::optional<at::Tensor> &dbetaInto) {
  checkBf16(dy, "dy");
  checkBf16(x, "x");
  c10::cuda::CUDAGuard g(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  auto dx = at::empty_like(x);
  // with both targets given the parameter gradients are added to them (they are the parameters' .grad)
  const bool into = dgammaInto.has_value() && dgammaInto->defined() && dbetaInto.has_value() && dbetaInto->defined();
  if (into) {
    checkBf16(*dgammaInto, "dgamma_into");
    checkBf16(*dbetaInto, "dbeta_into");
    TORCH_CHECK(dgammaInto->numel() == C && dbetaInto->numel() == C, "gradient targets must have one element per column");
  }
  auto dgamma = into ? *dgammaInto : at::empty_like(gamma), dbeta = into ? *dbetaInto : at::empty_like(gamma);
  auto partial = at::empty({fcxLnPartials(M), 2, C}, x.options().dtype(at::kFloat));
  const void *dr = dres.has_value() && dres->defined() ? dres->data_ptr() : nullptr;
  CUDA_OK(fcxLayerNormBwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), dr,
                          dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), partial.data_ptr<float>(), M, C, into ? 1 : 0, cur()));
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
static std::tuple<at::Tensor, at::Tensor> biasGeluBwd(const at::Tensor &dy, const at::Tensor &x, const at::Tensor &bias,
                                                        const c10::optional<at::Tensor> &dbiasInto) {
  checkBf16(dy, "dy");
  checkBf16(x, "x");
  c10::cuda::CUDAGuard g(x.device());
  const int C = (int)x.size(-1), M = (int)(x.numel() / C);
  auto dx = at::empty_like(x);
  CUDA_OK(fcxBiasGeluBwd(dy.data_ptr(), x.data_ptr(), bias.data_ptr(), dx.data_ptr(), M, C, cur()));
  const bool into = dbiasInto.has_value() && dbiasInto->defined();
  if (into) {
    checkBf16(*dbiasInto, "dbias_into");
    TORCH_CHECK(dbiasInto->numel() == C, "dbias_into must have one element per column");
  }
  auto dbias = into ? *dbiasInto : at::empty_like(bias);
  auto partial = at::empty({fcxColSumPartials(M), C}, x.options().dtype(at::kFloat));
  CUDA_OK(fcxColSum(dx.data_ptr(), dbias.data_ptr(), partial.data_ptr<float>(), M, C, into ? 1 : 0, cur()));
  return {dx, dbias};
}

static at::Tensor colSum(const at::Tensor &a, const c10::optional<at::Tensor> &intoT) {
  checkBf16(a, "a");
  c10::cuda::CUDAGuard g(a.device());
  const int C = (int)a.size(-1), M = (int)(a.numel() / C);
  const bool into = intoT.has_value() && intoT->defined();
  if (into) {
    checkBf16(*intoT, "into");
    TORCH_CHECK(intoT->numel() == C, "into must have one element per column");
  }
  auto out = into ? *intoT : at::empty({C}, a.options());
  auto partial = at::empty({fcxColSumPartials(M), C}, a.options().dtype(at::kFloat));
  CUDA_OK(fcxColSum(a.data_ptr(), out.data_ptr(), partial.data_ptr<float>(), M, C, into ? 1 : 0, cur()));
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
                  double eps, double wd, int64_t step, double gradScale, bool zeroGrad, const c10::optional<at::Tensor> &stepDev) {
  TORCH_CHECK(master.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat, "fp32 state");
  checkBf16(param, "param");
  checkBf16(grad, "grad");
  c10::cuda::CUDAGuard g(master.device());
  size_t n = master.numel();
  TORCH_CHECK((size_t)param.numel() == n && (size_t)grad.numel() == n && (size_t)m.numel() == n && (size_t)v.numel() == n, "size mismatch");
  CUDA_OK(fcxAdamW(master.data_ptr<float>(), param.data_ptr(), grad.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(), n, (float)lr,
                   (float)b1, (float)b2, (float)eps, (float)wd, (int)step, (float)gradScale, zeroGrad ? 1 : 0,
                   stepDev.has_value() && stepDev->defined() ? stepDev->data_ptr<int>() : nullptr, cur()));
}

// ---- direct access to a communicator from Python (raw flagcxComm_t as integer)

struct StreamLayout { cudaStream_t base; };

#define FCX_OK(call)                                                                                  \
  do {                                                                                                \
    flagcxResult_t _r = (call);                                                                       \
    TORCH_CHECK(_r == flagcxSuccess, "flagcx: ", flagcxGetErrorString(_r), ": ", flagcxGetLastError(nullptr)); \
  } while (0)

static flagcxDataType_t dtypeOf(const at::Tensor &t) {
  switch (t.scalar_type()) {
    case at::kChar: return flagcxInt8;
    case at::kByte: case at::kBool: return flagcxUint8;
    case at::kInt: return flagcxInt32;
    case at::kLong: return flagcxInt64;
    case at::kHalf: return flagcxFloat16;
    case at::kFloat: return flagcxFloat32;
    case at::kDouble: return flagcxFloat64;
    case at::kBFloat16: return flagcxBfloat16;
    case at::kFloat8_e4m3fn: return flagcxFloat8e4m3;
    case at::kFloat8_e5m2: return flagcxFloat8e5m2;
    default: TORCH_CHECK(false, "unsupported dtype");
  }
}

// A tensor whose storage lives in the communicator's symmetric heap.
static at::Tensor heapTensor(uint64_t comm, std::vector<int64_t> sizes, at::ScalarType dtype) {
  flagcxComm_t c = (flagcxComm_t)(uintptr_t)comm;
  int64_t numel = 1;
  for (auto s : sizes) numel *= s;
  size_t bytes = (size_t)numel * c10::elementSize(dtype);
  void *p = nullptr;
  FCX_OK(flagcxMemAlloc(&p, std::max<size_t>(bytes, 16), c));
  int dev = 0;
  flagcxCommGetDeviceNumber(c, &dev);
  // the tensor may outlive the communicator: it holds a reference that keeps the heap mapped until it dies
  FCX_OK(flagcxCommHeapRetain(c));
  return at::from_blob(p, sizes, [c](void *q) { flagcxCommHeapRelease(c, q); },
                       at::TensorOptions().dtype(dtype).device(at::Device(at::kCUDA, (c10::DeviceIndex)dev)));
}

static void commAllReduce(uint64_t comm, const at::Tensor &send, at::Tensor &recv, int64_t op, double scale) {
  flagcxComm_t c = (flagcxComm_t)(uintptr_t)comm;
  StreamLayout st{cur()};
  if (recv.scalar_type() != send.scalar_type() || scale != 1.0)
    FCX_OK(flagcxAllReduceCast(send.data_ptr(), recv.data_ptr(), send.numel(), dtypeOf(send), dtypeOf(recv), (float)scale,
                               (flagcxRedOp_t)op, c, (flagcxStream_t)&st));
  else
    FCX_OK(flagcxAllReduce(send.data_ptr(), recv.data_ptr(), send.numel(), dtypeOf(send), (flagcxRedOp_t)op, c, (flagcxStream_t)&st));
}
static void commAllGather(uint64_t comm, const at::Tensor &send, at::Tensor &recv) {
  StreamLayout st{cur()};
  FCX_OK(flagcxAllGather(send.data_ptr(), recv.data_ptr(), send.numel(), dtypeOf(send), (flagcxComm_t)(uintptr_t)comm, (flagcxStream_t)&st));
}
static void commReduceScatter(uint64_t comm, const at::Tensor &send, at::Tensor &recv, int64_t op) {
  StreamLayout st{cur()};
  FCX_OK(flagcxReduceScatter(send.data_ptr(), recv.data_ptr(), recv.numel(), dtypeOf(send), (flagcxRedOp_t)op,
                             (flagcxComm_t)(uintptr_t)comm, (flagcxStream_t)&st));
}
static void commAlltoAll(uint64_t comm, const at::Tensor &send, at::Tensor &recv) {
  flagcxComm_t c = (flagcxComm_t)(uintptr_t)comm;
  int n = 1;
  flagcxCommCount(c, &n);
  StreamLayout st{cur()};
  FCX_OK(flagcxAlltoAll(send.data_ptr(), recv.data_ptr(), send.numel() / n, dtypeOf(send), c, (flagcxStream_t)&st));
}
// counts and displacements in elements, one entry per rank, host lists as in flagcxAlltoAllv
static void commAlltoAllv(uint64_t comm, const at::Tensor &send, std::vector<int64_t> scounts, std::vector<int64_t> sdispls, at::Tensor &recv,
                          std::vector<int64_t> rcounts, std::vector<int64_t> rdispls) {
  StreamLayout st{cur()};
  std::vector<size_t> sc(scounts.begin(), scounts.end()), sd(sdispls.begin(), sdispls.end()), rc(rcounts.begin(), rcounts.end()),
      rd(rdispls.begin(), rdispls.end());
  FCX_OK(flagcxAlltoAllv(send.data_ptr(), sc.data(), sd.data(), recv.data_ptr(), rc.data(), rd.data(), dtypeOf(send),
                         (flagcxComm_t)(uintptr_t)comm, (flagcxStream_t)&st));
}
static void commBroadcast(uint64_t comm, at::Tensor &t, int64_t root) {
  StreamLayout st{cur()};
  FCX_OK(flagcxBroadcast(t.data_ptr(), t.data_ptr(), t.numel(), dtypeOf(t), (int)root, (flagcxComm_t)(uintptr_t)comm, (flagcxStream_t)&st));
}
// A communicator of its own for a component that launches collectives on its own stream (a communicator
// serves one stream at a time).  Collective over `comm`; destroyed with it unless comm_destroy is called first.
static uint64_t commSplit(uint64_t comm, int64_t color, int64_t key, int64_t stageBytes, int64_t userBytes) {
  flagcxComm_t child = nullptr;
  FCX_OK(flagcxCommSplitSized((flagcxComm_t)(uintptr_t)comm, (int)color, (int)key, (size_t)stageBytes, (size_t)userBytes, &child));
  return (uint64_t)(uintptr_t)child;
}
static void commDestroy(uint64_t comm) { FCX_OK(flagcxCommDestroy((flagcxComm_t)(uintptr_t)comm)); }
static void commSetCtaBudget(uint64_t comm, int64_t n) { FCX_OK(flagcxCommSetCtaBudget((flagcxComm_t)(uintptr_t)comm, (int)n)); }
static void commSetZcMulticast(uint64_t comm, int64_t mode) { FCX_OK(flagcxCommSetZeroCopyMulticast((flagcxComm_t)(uintptr_t)comm, (int)mode)); }
static void commPin(uint64_t comm, const std::string &kind, int64_t nctas) {
  FCX_OK(flagcxTunerPin((flagcxComm_t)(uintptr_t)comm, kind.empty() ? nullptr : kind.c_str(), (int)nctas));
}
static std::pair<std::string, int> commQuery(uint64_t comm, int64_t op, int64_t bytes, const at::Tensor &like, bool zeroCopy) {
  char kind[64] = {0};
  int nctas = 0;
  double est = 0;
  FCX_OK(flagcxTunerQueryEx((flagcxComm_t)(uintptr_t)comm, (flagcxCommOp_t)op, (size_t)bytes, dtypeOf(like), flagcxSum, zeroCopy ? 1 : 0,
                            kind, sizeof kind, &nctas, &est));
  return {std::string(kind), nctas};
}

static py::dict commCounters(uint64_t comm) {
  flagcxCommCounters cc;
  FCX_OK(flagcxCommGetCounters((flagcxComm_t)(uintptr_t)comm, &cc));
  py::dict d;
  d["launches"] = cc.launches;
  py::list calls, kinds;
  for (int i = 0; i < flagcxNumCommOps; i++) calls.append(cc.calls[i]);
  for (int i = 0; i < 24; i++) kinds.append(cc.kindLaunches[i]);
  d["calls"] = calls;
  d["kind_launches"] = kinds;
  return d;
}

}  // namespace fcxt

PYBIND11_MODULE(_flagcx_torch, m) {
  m.doc() = "flagcx_b200 native PyTorch pieces: c10d backend 'flagcx' and fused sm_100a ops";
  fcxt::bindBackend(m);
  fcxt::bindFused(m);
  m.def("layernorm_fwd", &fcxt::layernormFwd, py::arg("x"), py::arg("delta"), py::arg("gamma"), py::arg("beta"), py::arg("eps") = 1e-5);
  m.def("layernorm_bwd", &fcxt::layernormBwd, py::arg("dy"), py::arg("x"), py::arg("gamma"), py::arg("mean"), py::arg("rstd"), py::arg("dres"),
        py::arg("dgamma_into") = py::none(), py::arg("dbeta_into") = py::none());
  m.def("bias_gelu_fwd", &fcxt::biasGeluFwd);
  m.def("bias_gelu_bwd", &fcxt::biasGeluBwd, py::arg("dy"), py::arg("x"), py::arg("bias"), py::arg("dbias_into") = py::none());
  m.def("col_sum", &fcxt::colSum, py::arg("a"), py::arg("into") = py::none());
  m.def("cross_entropy_", &fcxt::crossEntropy);
  m.def("adamw_", &fcxt::adamw, py::arg("master"), py::arg("param"), py::arg("grad"), py::arg("m"), py::arg("v"), py::arg("lr"),
        py::arg("b1"), py::arg("b2"), py::arg("eps"), py::arg("wd"), py::arg("step"), py::arg("grad_scale"), py::arg("zero_grad"),
        py::arg("step_dev") = py::none());
  m.def("heap_tensor", &fcxt::heapTensor, "tensor allocated in the symmetric heap of a communicator");
  m.def("comm_all_reduce", &fcxt::commAllReduce, py::arg("comm"), py::arg("send"), py::arg("recv"), py::arg("op") = 0, py::arg("scale") = 1.0);
  m.def("comm_all_gather", &fcxt::commAllGather);
  m.def("comm_reduce_scatter", &fcxt::commReduceScatter, py::arg("comm"), py::arg("send"), py::arg("recv"), py::arg("op") = 0);
  m.def("comm_all_to_all", &fcxt::commAlltoAll);
  m.def("comm_all_to_all_v", &fcxt::commAlltoAllv);
  m.def("comm_broadcast", &fcxt::commBroadcast);
  m.def("comm_counters", &fcxt::commCounters);
  m.def("comm_split", &fcxt::commSplit, py::arg("comm"), py::arg("color"), py::arg("key"), py::arg("stage_bytes") = 0,
        py::arg("user_bytes") = 0);
  m.def("comm_destroy", &fcxt::commDestroy);
  m.def("comm_set_cta_budget", &fcxt::commSetCtaBudget);
  m.def("comm_set_zc_multicast", &fcxt::commSetZcMulticast);
  m.def("comm_pin", &fcxt::commPin, py::arg("comm"), py::arg("kind"), py::arg("nctas") = 16);
  m.def("comm_query", &fcxt::commQuery, py::arg("comm"), py::arg("op"), py::arg("bytes"), py::arg("like"), py::arg("zero_copy") = false);
}
