// Bindings of the tcgen05 GEMM family (gemm_sm100.cu).
#include <torch/extension.h>
namespace fcxt {
void bindGemm(py::module &) {}
}  // namespace fcxt
