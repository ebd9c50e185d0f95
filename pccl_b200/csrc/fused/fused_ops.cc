// Torch bindings of the fused operators.
#include "fused_ops.h"

#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "../common/util.h"
#include "../engine/engine.h"
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

// Heap bases of every connected rank, from the process-wide engine.
gemm::PeerBases peer_bases() {
  Engine& e = Engine::instance();
  gemm::PeerBases b{};
  b.rank = e.rank();
  b.world = e.world();
  for (int r = 0; r < b.world; ++r) b.base[r] = e.context().heap().data(r);
  return b;
}

uint32_t* as_u32(torch::Tensor& t, int64_t min_elems, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt32 && t.is_contiguous() && t.numel() >= min_elems,
              what, " must be a contiguous CUDA int32 tensor of at least ", min_elems, " elements");
  return reinterpret_cast<uint32_t*>(t.data_ptr());
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
  // Fused GEMM -> reduce-scatter over the engine's ranks (see fused/gemm_host.h for the contract).
  f.def("gemm_reduce_scatter",
        [](const torch::Tensor& x, const torch::Tensor& w, torch::Tensor& out, int64_t recv_off, int64_t flags_off,
           torch::Tensor& block_counter, int64_t epoch, int ctas) {
          const gemm::MatrixDesc dx = as_matrix(x, "x"), dw = as_matrix(w, "w");
          TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.stride(1) == 1, "out must be row-major bf16");
          gemm::gemm_reduce_scatter(peer_bases(), dx, dw, static_cast<uint64_t>(recv_off),
                                    static_cast<uint64_t>(flags_off),
                                    as_u32(block_counter, (x.size(0) + 127) / 128, "block_counter"), out.data_ptr(),
                                    out.stride(0), static_cast<uint32_t>(epoch),
                                    c10::cuda::getCurrentCUDAStream().stream(), ctas);
        },
        py::arg("x"), py::arg("w"), py::arg("out"), py::arg("recv_off"), py::arg("flags_off"),
        py::arg("block_counter"), py::arg("epoch"), py::arg("ctas") = 0);
  // Fused all-gather -> GEMM; the gathered activations live in the symmetric heap at gathered_off.
  f.def("all_gather_gemm",
        [](int64_t gathered_off, int64_t m, int64_t k, const torch::Tensor& w, torch::Tensor& out, int64_t flags_off,
           torch::Tensor& ready, int64_t epoch, int copy_ctas, int ctas) {
          const gemm::MatrixDesc dw = as_matrix(w, "w");
          TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.stride(1) == 1, "out must be row-major bf16");
          gemm::all_gather_gemm(peer_bases(), static_cast<uint64_t>(gathered_off), static_cast<int>(m),
                                static_cast<int>(k), dw, static_cast<uint64_t>(flags_off),
                                as_u32(ready, (m + 127) / 128, "ready"), out.data_ptr(), out.stride(0),
                                static_cast<uint32_t>(epoch), c10::cuda::getCurrentCUDAStream().stream(), copy_ctas,
                                ctas);
        },
        py::arg("gathered_off"), py::arg("m"), py::arg("k"), py::arg("w"), py::arg("out"), py::arg("flags_off"),
        py::arg("ready"), py::arg("epoch"), py::arg("copy_ctas") = 20, py::arg("ctas") = 0);
  // Fused all-reduce + residual + RMSNorm over symmetric buffers.
  f.def("ar_residual_rmsnorm",
        [](int64_t x_off, int64_t y_off, int64_t res_off, int64_t flags_off, const torch::Tensor& gamma,
           torch::Tensor& cta_counter, int64_t tokens, int64_t hidden, double eps, int64_t epoch, bool use_nvls,
           int ctas) {
          TORCH_CHECK(gamma.is_cuda() && gamma.scalar_type() == torch::kBFloat16 && gamma.is_contiguous() &&
                          gamma.numel() == hidden, "gamma must be a contiguous bf16 CUDA vector of `hidden` elements");
          Engine& e = Engine::instance();
          uint8_t* mc = (use_nvls && e.nvlsActive()) ? e.context().heap().mc_base() : nullptr;
          gemm::ar_residual_rmsnorm(peer_bases(), mc, static_cast<uint64_t>(x_off), static_cast<uint64_t>(y_off),
                                    static_cast<uint64_t>(res_off), static_cast<uint64_t>(flags_off),
                                    gamma.data_ptr(), as_u32(cta_counter, 1, "cta_counter"),
                                    static_cast<int>(tokens), static_cast<int>(hidden), static_cast<float>(eps),
                                    static_cast<uint32_t>(epoch), c10::cuda::getCurrentCUDAStream().stream(), ctas);
        },
        py::arg("x_off"), py::arg("y_off"), py::arg("res_off"), py::arg("flags_off"), py::arg("gamma"),
        py::arg("cta_counter"), py::arg("tokens"), py::arg("hidden"), py::arg("eps"), py::arg("epoch"),
        py::arg("use_nvls") = true, py::arg("ctas") = 0);
  // Device-side error word of the GEMM family (0 = ok); synchronises.
  f.def("read_error", &gemm::read_error);
  f.def("clear_error", &gemm::clear_error);
}

}  // namespace pccl
