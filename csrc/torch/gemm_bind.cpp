// Bindings of the tcgen05 GEMM family (gemm_sm100.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "flagcx.h"
#include "flagcx_ext.h"
#include "gemm_fp8_sm100.h"
#include "gemm_sm100.h"

namespace fcxt {

FcxDevComm devComm(uint64_t comm);                       // fused_ops.cpp
size_t heapOffset(uint64_t comm, const at::Tensor &t);   // fused_ops.cpp

static void checkMat(const at::Tensor &t, const char *name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1, name, " must be a 2-D bf16 CUDA tensor with contiguous rows");
}

// c[M,N] = a[M,K] @ b[N,K]^T on the tcgen05 path.  err is an int32 device scalar that the kernel sets when a wait gives up.
static at::Tensor gemmNT(const at::Tensor &a, const at::Tensor &b, at::Tensor &err) {
  checkMat(a, "a");
  checkMat(b, "b");
  TORCH_CHECK(a.size(1) == b.size(1), "inner dimensions differ");
  c10::cuda::CUDAGuard g(a.device());
  auto c = at::empty({a.size(0), b.size(0)}, a.options());
  auto e = fcxGemmBf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)a.size(0), (int)b.size(0), (int)a.size(1), (int)a.stride(0),
                       (int)b.stride(0), (int)c.stride(0), err.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "tcgen05 GEMM launch failed: ", cudaGetErrorString(e));
  return c;
}

// General form on the tcgen05 path.  a_mn / b_mn say how an operand is stored: False = [M,K] / [N,K] (K contiguous),
// True = [K,M] / [K,N] (the operand is read transposed where it lies).  So, for y = x w^T with x [T,I], w [O,I]:
//   forward   y  = gemm(x,  w,  False, False, bias)      [T,O]
//   dgrad     dx = gemm(dy, w,  False, True)              [T,I]   (w is [K=O, N=I])
//   wgrad     dw = gemm(dy, x,  True,  True)              [O,I]   (dy is [K=T, M=O], x is [K=T, N=I])
// split_k = 0 lets the launcher cut K when the output has too few tiles to fill the GPU (wgrad: K = tokens).
static at::Tensor gemmEx(const at::Tensor &a, const at::Tensor &b, bool aMN, bool bMN, const c10::optional<at::Tensor> &bias, int64_t splitK,
                         at::Tensor &err, int64_t pair, const c10::optional<at::Tensor> &out, bool accumulate) {
  checkMat(a, "a");
  checkMat(b, "b");
  const int64_t M = aMN ? a.size(1) : a.size(0), Ka = aMN ? a.size(0) : a.size(1);
  const int64_t N = bMN ? b.size(1) : b.size(0), Kb = bMN ? b.size(0) : b.size(1);
  TORCH_CHECK(Ka == Kb, "inner dimensions differ: ", Ka, " vs ", Kb);
  const void *biasPtr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kBFloat16 && bias->is_contiguous() && bias->numel() == N, "bias must be bf16 [N]");
    biasPtr = bias->data_ptr();
  }
  c10::cuda::CUDAGuard g(a.device());
  at::Tensor c;
  if (out.has_value() && out->defined()) {
    c = *out;
    TORCH_CHECK(c.is_cuda() && c.scalar_type() == at::kBFloat16 && c.dim() == 2 && c.size(0) == M && c.size(1) == N && c.stride(1) == 1,
                "out must be a bf16 [M, N] CUDA matrix with contiguous rows");
  } else {
    TORCH_CHECK(!accumulate, "accumulate needs out");
    c = at::empty({M, N}, a.options());
  }
  FcxGemmOpts o{};
  o.aMN = aMN ? 1 : 0; o.bMN = bMN ? 1 : 0; o.bias = biasPtr; o.splitK = (int)splitK; o.accumulate = accumulate ? 1 : 0; o.pair = (int)pair;
  auto e = fcxGemmBf16Opts(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)Ka, (int)a.stride(0), (int)b.stride(0),
                           (int)c.stride(0), &o, err.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "tcgen05 GEMM failed: ", cudaGetErrorString(e), ": ", fcxGemmLastDetail());
  return c;
}

// (pre, act) = (a w^T, gelu_tanh(a w^T + bias)) in one kernel: the CTA-pair GEMM writes both from its epilogue.  pre is what
// the backward pass of bias + GELU needs; a [M,K], w [N,K], bias [N] or None.
static std::tuple<at::Tensor, at::Tensor> gemmBiasGelu(const at::Tensor &a, const at::Tensor &w, const c10::optional<at::Tensor> &bias,
                                                       at::Tensor &err) {
  checkMat(a, "a");
  checkMat(w, "w");
  const int64_t M = a.size(0), K = a.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K, "inner dimensions differ: ", K, " vs ", w.size(1));
  const void *biasPtr = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kBFloat16 && bias->is_contiguous() && bias->numel() == N, "bias must be bf16 [N]");
    biasPtr = bias->data_ptr();
  }
  c10::cuda::CUDAGuard g(a.device());
  auto pre = at::empty({M, N}, a.options()), act = at::empty({M, N}, a.options());
  FcxGemmOpts o{};
  o.bias = biasPtr; o.splitK = 1; o.pair = 1; o.geluOut = act.data_ptr();
  auto e = fcxGemmBf16Opts(a.data_ptr(), w.data_ptr(), pre.data_ptr(), (int)M, (int)N, (int)K, (int)a.stride(0), (int)w.stride(0),
                           (int)pre.stride(0), &o, err.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "tcgen05 GEMM + GELU failed: ", cudaGetErrorString(e), ": ", fcxGemmLastDetail());
  return {pre, act};
}

// y[M,N] = all_gather(x_local)[M,K] @ w[N,K]^T.  gathered: heap tensor [M,K]; flags: heap int64 tensor [M/128];
// epoch: 1-based use count of this (gathered, flags) pair.
static at::Tensor agGemm(uint64_t comm, const at::Tensor &xLocal, at::Tensor &gathered, at::Tensor &flags, const at::Tensor &w,
                         int64_t epoch, int64_t commCtas, at::Tensor &err) {
  checkMat(xLocal, "x_local");
  checkMat(w, "w");
  TORCH_CHECK(xLocal.is_contiguous() && gathered.is_contiguous(), "x_local and gathered must be contiguous");
  c10::cuda::CUDAGuard g(xLocal.device());
  FcxDevComm dc = devComm(comm);
  const int M = (int)xLocal.size(0) * dc.nranks, K = (int)xLocal.size(1), N = (int)w.size(0);
  TORCH_CHECK(gathered.numel() >= (int64_t)M * K && flags.numel() >= M / 128, "workspace too small");
  auto y = at::empty({M, N}, xLocal.options());
  auto e = fcxAgGemmBf16(&dc, xLocal.data_ptr(), gathered.data_ptr(), heapOffset(comm, gathered), heapOffset(comm, flags), w.data_ptr(),
                         y.data_ptr(), M, N, K, (int)w.stride(0), (int)y.stride(0), (uint64_t)epoch, (int)commCtas, err.data_ptr<int>(),
                         at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "fused all-gather GEMM launch failed: ", cudaGetErrorString(e));
  return y;
}

// out[M/n,N] = reduce_scatter(a[M,K] @ w[N,K]^T).  stage: heap bf16 tensor [n, M/n, N]; counters: heap int64 tensor
// [M/n/128 * ceil(N/256)]; epoch: 1-based use count of this (stage, counters) pair.
static at::Tensor gemmRs(uint64_t comm, const at::Tensor &a, const at::Tensor &w, at::Tensor &stage, at::Tensor &counters, int64_t epoch,
                         at::Tensor &err) {
  checkMat(a, "a");
  checkMat(w, "w");
  c10::cuda::CUDAGuard g(a.device());
  FcxDevComm dc = devComm(comm);
  const int M = (int)a.size(0), K = (int)a.size(1), N = (int)w.size(0);
  TORCH_CHECK(M % (dc.nranks * 128) == 0, "rows must be a multiple of 128 x ranks");
  TORCH_CHECK(stage.numel() >= (int64_t)M * N && counters.numel() >= (M / dc.nranks / 128) * ((N + 255) / 256), "workspace too small");
  auto out = at::empty({M / dc.nranks, N}, a.options());
  auto e = fcxGemmRsBf16(&dc, a.data_ptr(), w.data_ptr(), out.data_ptr(), heapOffset(comm, stage), heapOffset(comm, counters), M, N, K,
                         (int)a.stride(0), (int)w.stride(0), (int)out.stride(0), (uint64_t)epoch, err.data_ptr<int>(),
                         at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "fused GEMM reduce-scatter launch failed: ", cudaGetErrorString(e));
  return out;
}

// bf16 [M,K] -> (e4m3 [M,K], fp32 scales [K/128, M])
static std::tuple<at::Tensor, at::Tensor> quantFp8Act(const at::Tensor &x) {
  checkMat(x, "x");
  TORCH_CHECK(x.size(1) % 128 == 0, "K must be a multiple of 128");
  c10::cuda::CUDAGuard g(x.device());
  auto q = at::empty({x.size(0), x.size(1)}, x.options().dtype(at::kFloat8_e4m3fn));
  auto sa = at::empty({x.size(1) / 128, x.size(0)}, x.options().dtype(at::kFloat));
  auto e = fcxQuantFp8Act(x.data_ptr(), q.data_ptr(), sa.data_ptr<float>(), (int)x.size(0), (int)x.size(1), (int)x.stride(0),
                          at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "fp8 quantisation launch failed: ", cudaGetErrorString(e));
  return {q, sa};
}

// bf16 [N,K] -> (e4m3 [N,K], fp32 scales [ceil(N/128), K/128])
static std::tuple<at::Tensor, at::Tensor> quantFp8Weight(const at::Tensor &w) {
  checkMat(w, "w");
  TORCH_CHECK(w.size(1) % 128 == 0, "K must be a multiple of 128");
  c10::cuda::CUDAGuard g(w.device());
  auto q = at::empty({w.size(0), w.size(1)}, w.options().dtype(at::kFloat8_e4m3fn));
  auto sb = at::empty({(w.size(0) + 127) / 128, w.size(1) / 128}, w.options().dtype(at::kFloat));
  auto e = fcxQuantFp8Weight(w.data_ptr(), q.data_ptr(), sb.data_ptr<float>(), (int)w.size(0), (int)w.size(1), (int)w.stride(0),
                             at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "fp8 quantisation launch failed: ", cudaGetErrorString(e));
  return {q, sb};
}

// bf16 c[M,N] = dequant(aq, sa) @ dequant(bq, sb)^T with the scales applied per 128-deep slice of K on the tcgen05 path
static at::Tensor gemmFp8NT(const at::Tensor &aq, const at::Tensor &sa, const at::Tensor &bq, const at::Tensor &sb, at::Tensor &err) {
  TORCH_CHECK(aq.is_cuda() && aq.scalar_type() == at::kFloat8_e4m3fn && aq.is_contiguous() && bq.scalar_type() == at::kFloat8_e4m3fn &&
                  bq.is_contiguous() && aq.dim() == 2 && bq.dim() == 2 && aq.size(1) == bq.size(1),
              "aq [M,K] and bq [N,K] must be contiguous e4m3 matrices");
  const int M = (int)aq.size(0), N = (int)bq.size(0), K = (int)aq.size(1);
  TORCH_CHECK(sa.scalar_type() == at::kFloat && sa.is_contiguous() && sa.numel() == (int64_t)(K / 128) * M, "sa must be fp32 [K/128, M]");
  TORCH_CHECK(sb.scalar_type() == at::kFloat && sb.is_contiguous() && sb.numel() == (int64_t)((N + 127) / 128) * (K / 128),
              "sb must be fp32 [ceil(N/128), K/128]");
  c10::cuda::CUDAGuard g(aq.device());
  auto c = at::empty({M, N}, aq.options().dtype(at::kBFloat16));
  auto e = fcxGemmFp8Blockwise(aq.data_ptr(), sa.data_ptr<float>(), bq.data_ptr(), sb.data_ptr<float>(), c.data_ptr(), M, N, K, (int)c.stride(0),
                               err.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "fp8 GEMM launch failed: ", cudaGetErrorString(e));
  return c;
}

void bindGemm(py::module &m) {
  m.def("quant_fp8_act", &quantFp8Act);
  m.def("quant_fp8_weight", &quantFp8Weight);
  m.def("gemm_fp8_nt", &gemmFp8NT, "block-scaled e4m3 GEMM (1x128 activation scales, 128x128 weight scales) on tcgen05");
  m.def("gemm_nt", &gemmNT, "bf16 a[M,K] @ b[N,K]^T on tcgen05");
  m.def("gemm", &gemmEx, py::arg("a"), py::arg("b"), py::arg("a_mn") = false, py::arg("b_mn") = false, py::arg("bias") = py::none(),
        py::arg("split_k") = 0, py::arg("err"), py::arg("pair") = -1, py::arg("out") = py::none(), py::arg("accumulate") = false,
        "out: write the result there; accumulate: add it to what out holds (a gradient that collects contributions). "
        "bf16 GEMM on tcgen05 with either operand read K-major or MN-major, optional bias row; pair: -1 kernel chosen by shape, "
        "0 one-CTA kernel (128 x 256 tiles), 1 CTA-pair kernel (cta_group::2, 256 x 256 tiles)");
  m.def("gemm_bias_gelu", &gemmBiasGelu, py::arg("a"), py::arg("w"), py::arg("bias"), py::arg("err"),
        "(a w^T, gelu_tanh(a w^T + bias)) from one CTA-pair GEMM launch");
  m.def("ag_gemm", &agGemm);
  m.def("gemm_rs", &gemmRs);
}

}  // namespace fcxt
