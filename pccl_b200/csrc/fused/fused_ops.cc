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
        [](const torch::Tensor& a, const torch::Tensor& b, c10::optional<torch::Tensor> out, int ctas,
           int sms_per_tile) {
          const gemm::MatrixDesc da = as_matrix(a, "a"), db = as_matrix(b, "b");
          torch::Tensor c = out.has_value() ? *out : torch::empty({a.size(0), b.size(0)}, a.options());
          TORCH_CHECK(c.scalar_type() == torch::kBFloat16 && c.stride(1) == 1 && c.size(0) == a.size(0) &&
                          c.size(1) == b.size(0), "out has the wrong shape / dtype");
          gemm::gemm_bf16_nt(da, db, c.data_ptr(), c.stride(0), c10::cuda::getCurrentCUDAStream().stream(), ctas,
                             2000, sms_per_tile);
          return c;
        },
        py::arg("a"), py::arg("b"), py::arg("out") = py::none(), py::arg("ctas") = 0, py::arg("sms_per_tile") = 0);
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
           torch::Tensor& ready, int64_t epoch, int copy_ctas, int ctas, bool swiglu) {
          const gemm::MatrixDesc dw = as_matrix(w, "w");
          TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.stride(1) == 1, "out must be row-major bf16");
          TORCH_CHECK(out.size(0) == m && out.size(1) == (swiglu ? w.size(0) / 2 : w.size(0)),
                      "out must be [M, N_local] (or [M, N_local / 2] with swiglu)");
          gemm::all_gather_gemm(peer_bases(), static_cast<uint64_t>(gathered_off), static_cast<int>(m),
                                static_cast<int>(k), dw, static_cast<uint64_t>(flags_off),
                                as_u32(ready, (m + 127) / 128, "ready"), out.data_ptr(), out.stride(0),
                                static_cast<uint32_t>(epoch), c10::cuda::getCurrentCUDAStream().stream(), copy_ctas,
                                ctas, 2000, swiglu);
        },
        py::arg("gathered_off"), py::arg("m"), py::arg("k"), py::arg("w"), py::arg("out"), py::arg("flags_off"),
        py::arg("ready"), py::arg("epoch"), py::arg("copy_ctas") = 0, py::arg("ctas") = 0, py::arg("swiglu") = false);
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
  // Packet-protocol all-reduce (sum) for small messages; out may be the input tensor.
  f.def("allreduce_ll",
        [](const torch::Tensor& in, torch::Tensor& out, int64_t buf_off, int64_t capacity_bytes, int64_t epoch,
           c10::optional<torch::Tensor> error) {
          TORCH_CHECK(in.is_cuda() && out.is_cuda() && in.is_contiguous() && out.is_contiguous() &&
                          in.scalar_type() == out.scalar_type() && in.numel() == out.numel(),
                      "allreduce_ll: contiguous CUDA tensors of one dtype and size");
          int dtype = -1;
          if (in.scalar_type() == torch::kFloat32) dtype = 0;
          else if (in.scalar_type() == torch::kFloat16) dtype = 1;
          else if (in.scalar_type() == torch::kBFloat16) dtype = 2;
          TORCH_CHECK(dtype >= 0, "allreduce_ll: float32, float16 or bfloat16");
          gemm::allreduce_ll(peer_bases(), static_cast<uint64_t>(buf_off), static_cast<uint64_t>(capacity_bytes),
                             in.data_ptr(), out.data_ptr(), static_cast<uint64_t>(in.nbytes()), dtype,
                             static_cast<uint32_t>(epoch), c10::cuda::getCurrentCUDAStream().stream(), 2000,
                             error.has_value() ? as_u32(*error, 1, "error") : nullptr);
        },
        py::arg("input"), py::arg("output"), py::arg("buf_off"), py::arg("capacity_bytes"), py::arg("epoch"),
        py::arg("error") = py::none());
  // Packet-protocol reduce-scatter (1), all-gather (2), all-to-all (3); sizes follow the collective.
  f.def("collective_ll",
        [](int mode, const torch::Tensor& in, torch::Tensor& out, int64_t buf_off, int64_t capacity_bytes, int64_t epoch,
           c10::optional<torch::Tensor> error) {
          TORCH_CHECK(in.is_cuda() && out.is_cuda() && in.is_contiguous() && out.is_contiguous() &&
                          in.scalar_type() == out.scalar_type(), "collective_ll: contiguous CUDA tensors of one dtype");
          TORCH_CHECK(mode >= 1 && mode <= 3, "collective_ll: mode 1..3");
          int dtype = -1;
          if (in.scalar_type() == torch::kFloat32) dtype = 0;
          else if (in.scalar_type() == torch::kFloat16) dtype = 1;
          else if (in.scalar_type() == torch::kBFloat16) dtype = 2;
          TORCH_CHECK(dtype >= 0, "collective_ll: float32, float16 or bfloat16");
          const gemm::PeerBases peers = peer_bases();
          const int64_t part = mode == 2 ? in.nbytes() : out.nbytes() / (mode == 3 ? peers.world : 1);
          const int64_t want_in = mode == 2 ? part : part * peers.world;
          const int64_t want_out = mode == 1 ? part : part * peers.world;
          TORCH_CHECK(static_cast<int64_t>(in.nbytes()) == want_in && static_cast<int64_t>(out.nbytes()) == want_out,
                      "collective_ll: tensor sizes do not match the collective");
          gemm::collective_ll(mode, peers, static_cast<uint64_t>(buf_off), static_cast<uint64_t>(capacity_bytes),
                              in.data_ptr(), out.data_ptr(), static_cast<uint64_t>(part), dtype,
                              static_cast<uint32_t>(epoch), c10::cuda::getCurrentCUDAStream().stream(), 2000,
                              error.has_value() ? as_u32(*error, 1, "error") : nullptr);
        },
        py::arg("mode"), py::arg("input"), py::arg("output"), py::arg("buf_off"), py::arg("capacity_bytes"),
        py::arg("epoch"), py::arg("error") = py::none());
  // Fused push collectives (mode: 0 all-reduce, 1 reduce-scatter, 2 all-gather, 3 all-to-all).
  f.def("collective_push",
        [](int mode, const torch::Tensor& in, torch::Tensor& out, int64_t area_off, int64_t capacity_bytes,
           int64_t flags_off, torch::Tensor& counters, int64_t epoch, int ctas, c10::optional<torch::Tensor> error) {
          TORCH_CHECK(in.is_cuda() && out.is_cuda() && in.is_contiguous() && out.is_contiguous() &&
                          in.scalar_type() == out.scalar_type(), "collective_push: contiguous CUDA tensors of one dtype");
          TORCH_CHECK(mode >= 0 && mode <= 3, "collective_push: mode 0..3");
          int dtype = -1;
          if (in.scalar_type() == torch::kFloat32) dtype = 0;
          else if (in.scalar_type() == torch::kFloat16) dtype = 1;
          else if (in.scalar_type() == torch::kBFloat16) dtype = 2;
          TORCH_CHECK(dtype >= 0, "collective_push: float32, float16 or bfloat16");
          const gemm::PeerBases peers = peer_bases();
          const int64_t full = mode == gemm::kPushAllGather ? out.nbytes() : in.nbytes();
          const int64_t want_out = mode == gemm::kPushReduceScatter ? full / peers.world : full;
          const int64_t want_in = mode == gemm::kPushAllGather ? full / peers.world : full;
          TORCH_CHECK(static_cast<int64_t>(out.nbytes()) == want_out && static_cast<int64_t>(in.nbytes()) == want_in,
                      "collective_push: tensor sizes do not match the collective");
          gemm::collective_push(static_cast<gemm::PushMode>(mode), peers, static_cast<uint64_t>(area_off),
                                static_cast<uint64_t>(capacity_bytes), static_cast<uint64_t>(flags_off),
                                as_u32(counters, 2, "counters"), in.data_ptr(), out.data_ptr(),
                                static_cast<uint64_t>(full), dtype, static_cast<uint32_t>(epoch),
                                c10::cuda::getCurrentCUDAStream().stream(), ctas, 2000,
                                error.has_value() ? as_u32(*error, 1, "error") : nullptr);
        },
        py::arg("mode"), py::arg("input"), py::arg("output"), py::arg("area_off"), py::arg("capacity_bytes"),
        py::arg("flags_off"), py::arg("counters"), py::arg("epoch"), py::arg("ctas"), py::arg("error") = py::none());
  // In-switch all-reduce (sum) of `bytes` at a symmetric-heap offset, in place.
  f.def("allreduce_nvls",
        [](int64_t data_off, int64_t bytes, int dtype, int64_t flags_off, torch::Tensor& cta_counter, int64_t epoch,
           int ctas, c10::optional<torch::Tensor> error) {
          Engine& e = Engine::instance();
          TORCH_CHECK(e.nvlsActive(), "allreduce_nvls: the engine has no multicast mapping");
          gemm::allreduce_nvls(peer_bases(), e.context().heap().mc_base(), static_cast<uint64_t>(data_off),
                               static_cast<uint64_t>(bytes), dtype, static_cast<uint64_t>(flags_off),
                               as_u32(cta_counter, 1, "cta_counter"), static_cast<uint32_t>(epoch),
                               c10::cuda::getCurrentCUDAStream().stream(), ctas, 2000,
                               error.has_value() ? as_u32(*error, 1, "error") : nullptr);
        },
        py::arg("data_off"), py::arg("bytes"), py::arg("dtype"), py::arg("flags_off"), py::arg("cta_counter"),
        py::arg("epoch"), py::arg("ctas"), py::arg("error") = py::none());
  // MoE router on its own: top-2 expert indices, renormalised gates, the row each choice claims
  // in its expert's batch, and the per-expert token counts.  scratch: int32[experts + 1].
  f.def("moe_route",
        [](const torch::Tensor& x, const torch::Tensor& wg, torch::Tensor& scratch, torch::Tensor& topk_idx,
           torch::Tensor& topk_gate, torch::Tensor& topk_slot, torch::Tensor& counts) {
          const gemm::MatrixDesc dx = as_matrix(x, "x"), dg = as_matrix(wg, "wg");
          TORCH_CHECK(x.is_contiguous() && wg.is_contiguous() && dx.cols == dg.cols, "x / wg must be contiguous [*, hidden]");
          TORCH_CHECK(topk_gate.is_cuda() && topk_gate.scalar_type() == torch::kFloat32 && topk_gate.is_contiguous() &&
                          topk_gate.numel() >= 2 * dx.rows, "topk_gate must be float32 [tokens, 2]");
          gemm::PeerBases self{};
          self.rank = 0;
          self.world = 1;
          gemm::MoeBuffers none{};
          gemm::moe_route_dispatch(self, none, x.data_ptr(), wg.data_ptr(), dx.rows, dx.cols, dg.rows,
                                   as_u32(scratch, dg.rows + 1, "scratch"),
                                   reinterpret_cast<int32_t*>(as_u32(topk_idx, 2 * dx.rows, "topk_idx")),
                                   topk_gate.data_ptr<float>(),
                                   reinterpret_cast<int32_t*>(as_u32(topk_slot, 2 * dx.rows, "topk_slot")),
                                   as_u32(counts, dg.rows, "counts"), false, 1,
                                   c10::cuda::getCurrentCUDAStream().stream());
        },
        py::arg("x"), py::arg("wg"), py::arg("scratch"), py::arg("topk_idx"), py::arg("topk_gate"),
        py::arg("topk_slot"), py::arg("counts"));
  // Expert-parallel MoE feed-forward: route + dispatch, expert GEMM 1 (SwiGLU), expert GEMM 2 +
  // return + combine.  offsets = [recv, meta, counts, ready, done, comb] in the symmetric heap
  // (or in `local_heap`, a CUDA byte tensor standing in for it on a single GPU without an
  // engine).  phases: bit 0 dispatch, bit 1 up, bit 2 down (all three by default).
  f.def("moe_forward",
        [](const torch::Tensor& x, const torch::Tensor& wg, const torch::Tensor& w13, const torch::Tensor& w2,
           torch::Tensor& h, torch::Tensor& out, torch::Tensor& scratch, torch::Tensor& cta_counter,
           const std::vector<int64_t>& offsets, int64_t cap, int64_t epoch, c10::optional<torch::Tensor> local_heap,
           int ctas, int phases, c10::optional<torch::Tensor> topk_idx, c10::optional<torch::Tensor> topk_gate) {
          const gemm::MatrixDesc dx = as_matrix(x, "x"), dg = as_matrix(wg, "wg");
          const gemm::MatrixDesc d13 = as_matrix(w13, "w13"), d2 = as_matrix(w2, "w2");
          TORCH_CHECK(x.is_contiguous() && wg.is_contiguous() && w13.is_contiguous() && w2.is_contiguous() &&
                          h.is_contiguous() && out.is_contiguous(), "MoE operands must be contiguous");
          TORCH_CHECK(offsets.size() == 6, "offsets = [recv, meta, counts, ready, done, comb]");
          gemm::PeerBases peers{};
          if (local_heap.has_value()) {
            TORCH_CHECK(local_heap->is_cuda() && local_heap->is_contiguous(), "local_heap must be a CUDA buffer");
            peers.rank = 0;
            peers.world = 1;
            peers.base[0] = static_cast<uint8_t*>(local_heap->data_ptr());
          } else {
            peers = peer_bases();
          }
          const int tokens = dx.rows, hidden = dx.cols, experts = dg.rows;
          TORCH_CHECK(experts % peers.world == 0, "experts must divide over the ranks");
          const int local_experts = experts / peers.world;
          const int ffn = d2.cols;
          TORCH_CHECK(d13.rows == local_experts * 2 * ffn && d13.cols == hidden, "w13 must be [local_experts * 2 * ffn, hidden]");
          TORCH_CHECK(d2.rows == local_experts * hidden, "w2 must be [local_experts * hidden, ffn]");
          TORCH_CHECK(cap >= tokens, "region capacity must cover the tokens of one rank");
          TORCH_CHECK(h.scalar_type() == torch::kBFloat16 &&
                          h.numel() >= static_cast<int64_t>(local_experts) * peers.world * cap * ffn, "h is too small");
          TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.numel() == static_cast<int64_t>(tokens) * hidden,
                      "out must be bf16 [tokens, hidden]");
          gemm::MoeBuffers buf{};
          buf.recv_off = offsets[0]; buf.meta_off = offsets[1]; buf.counts_off = offsets[2];
          buf.ready_off = offsets[3]; buf.done_off = offsets[4]; buf.comb_off = offsets[5];
          buf.cap = static_cast<int>(cap);
          cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
          int32_t* idx = topk_idx.has_value() ? reinterpret_cast<int32_t*>(as_u32(*topk_idx, 2 * tokens, "topk_idx")) : nullptr;
          float* gate = nullptr;
          if (topk_gate.has_value()) {
            TORCH_CHECK(topk_gate->is_cuda() && topk_gate->scalar_type() == torch::kFloat32 &&
                            topk_gate->is_contiguous() && topk_gate->numel() >= 2 * tokens, "topk_gate must be float32 [tokens, 2]");
            gate = topk_gate->data_ptr<float>();
          }
          if (phases & 1)
            gemm::moe_route_dispatch(peers, buf, x.data_ptr(), wg.data_ptr(), tokens, hidden, experts,
                                     as_u32(scratch, experts + 1, "scratch"), idx, gate, nullptr, nullptr, true,
                                     static_cast<uint32_t>(epoch), stream);
          if (phases & 2)
            gemm::moe_expert_up(peers, buf, hidden, ffn, local_experts, w13.data_ptr(), h.data_ptr(),
                                static_cast<uint32_t>(epoch), stream, ctas);
          if (phases & 4)
            gemm::moe_expert_down(peers, buf, tokens, hidden, ffn, local_experts, h.data_ptr(), w2.data_ptr(),
                                  out.data_ptr(), as_u32(cta_counter, 1, "cta_counter"),
                                  static_cast<uint32_t>(epoch), stream, ctas);
        },
        py::arg("x"), py::arg("wg"), py::arg("w13"), py::arg("w2"), py::arg("h"), py::arg("out"), py::arg("scratch"),
        py::arg("cta_counter"), py::arg("offsets"), py::arg("cap"), py::arg("epoch"),
        py::arg("local_heap") = py::none(), py::arg("ctas") = 0, py::arg("phases") = 7,
        py::arg("topk_idx") = py::none(), py::arg("topk_gate") = py::none());
  // Gather a list of contiguous tensors into `bucket` at the given byte offsets (unpack: scatter back).
  f.def("bucket_pack",
        [](const std::vector<torch::Tensor>& tensors, const std::vector<int64_t>& offsets, torch::Tensor& bucket,
           bool unpack) {
          TORCH_CHECK(tensors.size() == offsets.size(), "one offset per tensor");
          TORCH_CHECK(bucket.is_cuda() && bucket.is_contiguous(), "bucket must be a contiguous CUDA tensor");
          std::vector<gemm::PackEntry> entries;
          entries.reserve(tensors.size());
          for (size_t i = 0; i < tensors.size(); ++i) {
            const torch::Tensor& t = tensors[i];
            TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "bucket_pack: tensors must be contiguous CUDA tensors");
            TORCH_CHECK(offsets[i] >= 0 && offsets[i] + static_cast<int64_t>(t.nbytes()) <= static_cast<int64_t>(bucket.nbytes()),
                        "bucket_pack: tensor ", i, " does not fit the bucket at offset ", offsets[i]);
            entries.push_back({t.data_ptr(), static_cast<uint64_t>(offsets[i]), static_cast<uint64_t>(t.nbytes())});
          }
          gemm::bucket_pack(entries.data(), static_cast<int>(entries.size()), bucket.data_ptr(), unpack,
                            c10::cuda::getCurrentCUDAStream().stream());
        },
        py::arg("tensors"), py::arg("offsets"), py::arg("bucket"), py::arg("unpack") = false);
  // Per-CTA milestones of the most recent GEMM-family launch (see gemm_host.h).
  f.def("gemm_trace_enable", &gemm::gemm_trace_enable);
  f.def("gemm_trace_read", &gemm::gemm_trace_read);
  // Device-side error word of the GEMM family (0 = ok); synchronises.
  f.def("read_error", &gemm::read_error);
  f.def("clear_error", &gemm::clear_error);
}

}  // namespace pccl
