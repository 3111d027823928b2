// Bindings of the expert-parallel MoE kernels (moe_sm100.cu) and of the GEMM variants they use.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "flagcx.h"
#include "flagcx_ext.h"
#include "gemm_sm100.h"
#include "moe_sm100.h"

namespace fcxt {

FcxDevComm devComm(uint64_t comm);                       // fused_ops.cpp
size_t heapOffset(uint64_t comm, const at::Tensor &t);   // fused_ops.cpp

static cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }

static void checkBf16Mat(const at::Tensor &t, const char *name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1, name,
              " must be a 2-D bf16 CUDA tensor with contiguous rows");
}

// Route this rank's tokens to their experts.  All heap tensors belong to one buffer set; epoch is that set's 1-based use count.
static void moeDispatch(uint64_t comm, const at::Tensor &x, const at::Tensor &topkIdx, at::Tensor &countMat, at::Tensor &countFlags,
                        at::Tensor &recv, at::Tensor &info, at::Tensor &done, int64_t epoch, at::Tensor &slot, at::Tensor &localCounts,
                        at::Tensor &recvTotal, at::Tensor &err, int64_t ctas, int64_t expertsPerRank) {
  checkBf16Mat(x, "x");
  TORCH_CHECK(x.is_contiguous() && topkIdx.is_contiguous() && topkIdx.scalar_type() == at::kInt && topkIdx.dim() == 2, "topk_idx must be int32 [T, K]");
  TORCH_CHECK(topkIdx.size(0) == x.size(0), "topk_idx and x disagree on the token count");
  c10::cuda::CUDAGuard g(x.device());
  FcxDevComm dc = devComm(comm);
  FcxMoeParams p{};
  p.x = x.data_ptr();
  p.topkIdx = topkIdx.data_ptr<int>();
  p.T = (int)x.size(0);
  p.H = (int)x.size(1);
  p.K = (int)topkIdx.size(1);
  p.cap = (int)recv.size(0);
  p.L = (int)expertsPerRank;
  TORCH_CHECK(p.L >= 1 && dc.nranks * p.L <= 64 && p.cap % p.L == 0, "experts_per_rank: 1..64/nranks, dividing the buffer rows");
  TORCH_CHECK(recv.size(1) == p.H && info.numel() >= (int64_t)p.cap * 4 && countMat.numel() >= (int64_t)dc.nranks * dc.nranks * p.L &&
                  countFlags.numel() >= dc.nranks && done.numel() >= dc.nranks && slot.numel() >= (int64_t)p.T * p.K &&
                  localCounts.numel() >= dc.nranks * p.L && recvTotal.numel() >= p.L,
              "workspace too small");
  p.countMatOff = heapOffset(comm, countMat);
  p.countFlagOff = heapOffset(comm, countFlags);
  p.recvOff = heapOffset(comm, recv);
  p.infoOff = heapOffset(comm, info);
  p.doneOff = heapOffset(comm, done);
  p.epoch = (uint64_t)epoch;
  p.slot = slot.data_ptr<int>();
  p.localCounts = localCounts.data_ptr<int>();
  p.recvTotal = recvTotal.data_ptr<int>();
  p.errFlag = err.data_ptr<int>();
  auto e = fcxMoeDispatch(&dc, &p, (int)ctas, cur());
  TORCH_CHECK(e == cudaSuccess, "MoE dispatch launch failed: ", cudaGetErrorString(e));
}

static void siluMul(const at::Tensor &gu, at::Tensor &h, const c10::optional<at::Tensor> &rows) {
  checkBf16Mat(gu, "gu");
  checkBf16Mat(h, "h");
  TORCH_CHECK(gu.is_contiguous() && h.is_contiguous() && gu.size(1) == 2 * h.size(1) && gu.size(0) == h.size(0), "gu must be [R, 2F] and h [R, F]");
  c10::cuda::CUDAGuard g(gu.device());
  auto e = fcxSiluMul(gu.data_ptr(), h.data_ptr(), rows ? rows->data_ptr<int>() : nullptr, (int)h.size(0), (int)h.size(1), cur());
  TORCH_CHECK(e == cudaSuccess, "silu_mul launch failed: ", cudaGetErrorString(e));
}

// c[:*m_ptr] = a[:*m_ptr] @ b^T; rows beyond *m_ptr are left untouched.
static void gemmDynM(const at::Tensor &a, const at::Tensor &b, at::Tensor &c, const at::Tensor &mPtr, at::Tensor &err) {
  checkBf16Mat(a, "a");
  checkBf16Mat(b, "b");
  checkBf16Mat(c, "c");
  TORCH_CHECK(a.size(1) == b.size(1) && c.size(0) == a.size(0) && c.size(1) == b.size(0), "shape mismatch");
  c10::cuda::CUDAGuard g(a.device());
  auto e = fcxGemmBf16DynM(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)a.size(0), mPtr.data_ptr<int>(), (int)b.size(0), (int)a.size(1),
                           (int)a.stride(0), (int)b.stride(0), (int)c.stride(0), err.data_ptr<int>(), cur());
  TORCH_CHECK(e == cudaSuccess, "tcgen05 GEMM launch failed: ", cudaGetErrorString(e));
}

// Expert output projection whose epilogue returns every row to the rank the token came from.  Returns the grid size:
// each of its CTAs adds 1 to done_counter on every rank.
static int64_t gemmRowMap(uint64_t comm, const at::Tensor &a, const at::Tensor &b, const at::Tensor &mPtr, const at::Tensor &info,
                          at::Tensor &combine, at::Tensor &doneCounter, int64_t topk, at::Tensor &err) {
  checkBf16Mat(a, "a");
  checkBf16Mat(b, "b");
  TORCH_CHECK(a.size(1) == b.size(1), "inner dimensions differ");
  TORCH_CHECK(info.scalar_type() == at::kInt && info.numel() >= a.size(0) * 4, "info must be int32 [rows, 4]");
  c10::cuda::CUDAGuard g(a.device());
  FcxDevComm dc = devComm(comm);
  int grid = 0;
  auto e = fcxGemmRowMapBf16(&dc, a.data_ptr(), b.data_ptr(), (int)a.size(0), mPtr.data_ptr<int>(), (int)b.size(0), (int)a.size(1),
                             (int)a.stride(0), (int)b.stride(0), info.data_ptr(), heapOffset(comm, combine), heapOffset(comm, doneCounter),
                             (int)topk, err.data_ptr<int>(), &grid, cur());
  TORCH_CHECK(e == cudaSuccess, "fused GEMM combine launch failed: ", cudaGetErrorString(e));
  return grid;
}

static void moeCombine(uint64_t comm, const at::Tensor &combine, const at::Tensor &topkW, at::Tensor &out, const at::Tensor &doneCounter,
                       int64_t want, at::Tensor &err) {
  checkBf16Mat(out, "out");
  TORCH_CHECK(topkW.scalar_type() == at::kFloat && topkW.is_contiguous() && topkW.dim() == 2 && out.is_contiguous(), "topk_w must be fp32 [T, K]");
  const int T = (int)out.size(0), H = (int)out.size(1), K = (int)topkW.size(1);
  TORCH_CHECK(combine.numel() >= (int64_t)T * K * H, "combine buffer too small");
  c10::cuda::CUDAGuard g(out.device());
  FcxDevComm dc = devComm(comm);
  auto e = fcxMoeCombine(&dc, combine.data_ptr(), topkW.data_ptr<float>(), out.data_ptr(), T, H, K, heapOffset(comm, doneCounter),
                         (uint64_t)want, err.data_ptr<int>(), cur());
  TORCH_CHECK(e == cudaSuccess, "MoE combine launch failed: ", cudaGetErrorString(e));
}

void bindMoe(py::module &m) {
  m.def("moe_dispatch", &moeDispatch, py::arg("comm"), py::arg("x"), py::arg("topk_idx"), py::arg("count_mat"), py::arg("count_flags"),
        py::arg("recv"), py::arg("info"), py::arg("done"), py::arg("epoch"), py::arg("slot"), py::arg("local_counts"), py::arg("recv_total"),
        py::arg("err"), py::arg("ctas"), py::arg("experts_per_rank") = 1);
  m.def("silu_mul", &siluMul, py::arg("gu"), py::arg("h"), py::arg("rows") = py::none());
  m.def("gemm_dyn_m", &gemmDynM);
  m.def("gemm_rowmap", &gemmRowMap);
  m.def("moe_combine", &moeCombine);
}

}  // namespace fcxt
