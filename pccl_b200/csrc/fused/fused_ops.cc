// Torch bindings of the fused operators.
#include "fused_ops.h"

#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "../common/util.h"
#include "gemm_host.h"

namespace py = pybind11;

namespace pccl {

namespace {

gemm::MatrixDesc as_matrix(const torch::Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 2, what, " must be a 2-D CUDA tensor");
  TORCH_CHECK(t.scalar_type() == torch::kBFloat16, what, " must be bfloat16");
  TORCH_CHECK(t.stride(1) == 1, what, " must be row-major (unit stride in the last dimension)");
  return gemm::MatrixDesc{t.data_ptr(), static_cast<int>(t.size(0)), static_cast<int>(t.size(1)), t.stride(0)};
}

}  // namespace

void bind_fused_ops(py::module_& m) {
  auto f = m.def_submodule("fused", "tcgen05 / TMEM fused operators");
  // c[M,N] = a[M,K] @ b[N,K]^T   (nn.Linear weight layout), bf16 in / bf16 out, fp32 accumulate.
  f.def("matmul_nt",
        [](const torch::Tensor& a, const torch::Tensor& b, c10::optional<torch::Tensor> out, int ctas) {
          const gemm::MatrixDesc da = as_matrix(a, "a"), db = as_matrix(b, "b");
          torch::Tensor c = out.has_value() ? *out : torch::empty({a.size(0), b.size(0)}, a.options());
          TORCH_CHECK(c.scalar_type() == torch::kBFloat16 && c.stride(1) == 1 && c.size(0) == a.size(0) &&
                          c.size(1) == b.size(0), "out has the wrong shape / dtype");
          gemm::gemm_bf16_nt(da, db, c.data_ptr(), c.stride(0), c10::cuda::getCurrentCUDAStream().stream(), ctas);
          return c;
        },
        py::arg("a"), py::arg("b"), py::arg("out") = py::none(), py::arg("ctas") = 0);
  // Device-side error word of the GEMM family (0 = ok); synchronises.
  f.def("read_error", &gemm::read_error);
  f.def("clear_error", &gemm::clear_error);
}

}  // namespace pccl
