// Python bindings of the kernels that communicate from inside the kernel:
// the device-API ring exchange, and (gemm_*.cu) the fused GEMM + collective kernels.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "flagcx.h"
#include "flagcx_ext.h"
#include "../kernels/devcomm.h"

extern "C" cudaError_t fcxRingExchange(const FcxDevComm *dc, const void *src, size_t inboxOffset, void *dst, size_t bytes, int slot,
                                       unsigned long long epoch, int *status, int nblocks, cudaStream_t s);

namespace fcxt {

#define FCX_OK2(call)                                                                               \
  do {                                                                                              \
    flagcxResult_t _r = (call);                                                                     \
    TORCH_CHECK(_r == flagcxSuccess, "flagcx: ", flagcxGetErrorString(_r), ": ", flagcxGetLastError(nullptr)); \
  } while (0)

FcxDevComm devComm(uint64_t comm) {
  FcxDevComm dc;
  FCX_OK2(flagcxCommDeviceDescriptor((flagcxComm_t)(uintptr_t)comm, &dc, sizeof dc));
  return dc;
}

size_t heapOffset(uint64_t comm, const at::Tensor &t) {
  size_t off = 0;
  FCX_OK2(flagcxHeapOffset((flagcxComm_t)(uintptr_t)comm, t.data_ptr(), &off));
  return off;
}

// dst <- the block that the previous rank of the ring holds in src.  `inbox` must be a heap tensor
// (flagcx_b200.native().heap_tensor) at least as large as src; `epoch` counts calls on this slot from 1.
static void ringExchange(uint64_t comm, const at::Tensor &src, at::Tensor &inbox, at::Tensor &dst, int64_t slot, int64_t epoch) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && dst.is_contiguous() && inbox.is_contiguous(), "contiguous CUDA tensors");
  TORCH_CHECK(inbox.nbytes() >= src.nbytes() && dst.nbytes() >= src.nbytes(), "inbox and dst must hold the message");
  c10::cuda::CUDAGuard g(src.device());
  FcxDevComm dc = devComm(comm);
  auto status = at::zeros({1}, src.options().dtype(at::kInt));
  int nblocks = (int)std::max<int64_t>(1, std::min<int64_t>(32, (int64_t)src.nbytes() / (256 << 10)));
  auto e = fcxRingExchange(&dc, src.data_ptr(), heapOffset(comm, inbox), dst.data_ptr(), src.nbytes(), (int)slot,
                           (unsigned long long)epoch, status.data_ptr<int>(), nblocks, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(e == cudaSuccess, "ring exchange launch failed: ", cudaGetErrorString(e));
}

static int64_t allocSignals(uint64_t comm, int64_t n) {
  int first = 0;
  FCX_OK2(flagcxCommAllocSignals((flagcxComm_t)(uintptr_t)comm, (int)n, &first));
  return first;
}

void bindGemm(py::module &m);  // gemm_bind.cpp
void bindMoe(py::module &m);   // moe_bind.cpp

void bindFused(py::module &m) {
  m.def("ring_exchange", &ringExchange, py::arg("comm"), py::arg("src"), py::arg("inbox"), py::arg("dst"), py::arg("slot"), py::arg("epoch"));
  m.def("alloc_signals", &allocSignals);
  bindGemm(m);
  bindMoe(m);
}

}  // namespace fcxt
