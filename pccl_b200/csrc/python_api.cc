// Python bindings: module pccl_b200.engine_c (also importable as pccl.engine_c).
// Method names on Engine follow the reference's binding (reference:
// csrc/python_api.cc:11-33) so the Python wrapper's calls are unchanged; everything
// else (status, reset, NVLS stages, symmetric tensors, LocalCluster, fused
// operators) is an addition.
#include <c10/cuda/CUDAStream.h>
#include <execinfo.h>
#include <signal.h>
#include <unistd.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "common/launch.h"
#include "common/util.h"
#include "engine/engine.h"
#include "fused/fused_ops.h"
#include "ocs/signal_board.h"
namespace pccl { void bind_rdma(pybind11::module_& m); }

namespace py = pybind11;
using namespace pccl;

namespace {

cudaStream_t current_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

void check_tensor(const torch::Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda(), what, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), what, " must be contiguous");
}

void exe(const std::string& name, const torch::Tensor& in, torch::Tensor& out, bool sync) {
  check_tensor(in, "input");
  check_tensor(out, "output");
  Engine::instance().exeOp(name, in.data_ptr(), in.nbytes(), out.data_ptr(), out.nbytes(), current_stream(), sync);
}

// A tensor that aliases symmetric memory; the engine owns the storage.
torch::Tensor heap_tensor(uint8_t* base, const std::vector<int64_t>& shape, torch::ScalarType dtype, int device) {
  auto options = torch::TensorOptions().dtype(dtype).device(torch::kCUDA, device);
  return torch::from_blob(base, shape, [](void*) {}, options);
}

// PCCL_BACKTRACE=1: print the native stack on SIGSEGV before the default action.
void segv_backtrace(int sig) {
  void* frames[64];
  const int n = backtrace(frames, 64);
  backtrace_symbols_fd(frames, n, STDERR_FILENO);
  signal(sig, SIG_DFL);
  raise(sig);
}

int64_t numel_of(const std::vector<int64_t>& shape) {
  int64_t n = 1;
  for (int64_t e : shape) n *= e;
  return n;
}

py::list trace_list(RankContext& ctx, const std::string& name) {
  static const char* kinds[] = {"noop", "copy", "reduce", "put", "reduce_multi", "multimem.reduce",
                                "multimem.store", "multimem.allreduce", "scale"};
  py::list out;
  for (const TraceStep& t : ctx.read_trace(ctx.op(name))) {
    py::dict d;
    d["chain"] = t.chain; d["step"] = t.step; d["kind"] = kinds[t.kind < 9 ? t.kind : 0];
    d["ctas"] = t.ctas; d["bytes"] = t.bytes;
    d["t_reached_ns"] = t.t[0]; d["t_data_ns"] = t.t[1]; d["t_done_ns"] = t.t[2]; d["t_posted_ns"] = t.t[3];
    out.append(d);
  }
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "pccl_b200 native engine";
  m.attr("version") = "0.3.0";
  if (Environs::get_flag("PCCL_BACKTRACE")) signal(SIGSEGV, segv_backtrace);
  py::register_exception<Error>(m, "PCCLError", PyExc_RuntimeError);
  py::register_exception<TimeoutError>(m, "PCCLTimeoutError", m.attr("PCCLError").ptr());

  py::class_<Engine, std::unique_ptr<Engine, py::nodelete>>(m, "Engine")
      .def_static("get_instance", &Engine::instance, py::return_value_policy::reference)
      .def("regOp", &Engine::regOp)
      .def("regOpFromString", &Engine::regOpFromString)
      .def("exeOp", [](Engine&, const std::string& n, const torch::Tensor& i, torch::Tensor& o) { exe(n, i, o, true); })
      .def("exeOpAsync", [](Engine&, const std::string& n, const torch::Tensor& i, torch::Tensor& o) { exe(n, i, o, false); })
      .def("syncOp", [](Engine& e, const std::string& n) { e.syncOp(n, current_stream()); })
      .def("resetSignals", &Engine::resetSignals)
      .def("reset", &Engine::reset)
      .def("exportEndpoint", &Engine::exportEndpoint)
      .def("updateEndpoint", &Engine::updateEndpoint)
      .def("nvlsStage", &Engine::nvlsStage)
      .def("nvlsDisable", &Engine::nvlsDisable)
      .def("nvlsActive", &Engine::nvlsActive)
      .def("rank", &Engine::rank)
      .def("world", &Engine::world)
      .def("stats", &Engine::statsJson)
      .def("setTimeoutMs", [](Engine& e, uint64_t ms) { e.context().set_timeout_ms(ms); })
      // Device timeline: setTrace(True), run, synchronize, then trace(name) lists every step of the
      // last launch with its four %globaltimer stamps (ns since the launch's first stamp).
      .def("setTrace", [](Engine& e, bool on) { e.context().set_trace(on); })
      .def("trace", [](Engine& e, const std::string& name) { return trace_list(e.context(), name); })
      .def("bufferBytes", [](Engine& e) { return e.context().buffer_bytes(); })
      // View of the plan working buffer: collectives on it run without staging copies.
      .def("workingBuffer",
           [](Engine& e, const std::vector<int64_t>& shape, torch::ScalarType dtype, int64_t offset_bytes) {
             RankContext& c = e.context();
             const int64_t bytes = numel_of(shape) * static_cast<int64_t>(c10::elementSize(dtype));
             TORCH_CHECK(offset_bytes >= 0 && offset_bytes + bytes <= static_cast<int64_t>(c.buffer_bytes()),
                         "working-buffer view exceeds PCCL_BUFFER_SIZE");
             return heap_tensor(c.heap().data(c.rank()) + offset_bytes, shape, dtype, c.heap().device());
           },
           py::arg("shape"), py::arg("dtype"), py::arg("offset_bytes") = 0)
      // Symmetric allocation from the arena (same offset on every rank when all allocate alike).
      .def("allocSymmetric",
           [](Engine& e, const std::vector<int64_t>& shape, torch::ScalarType dtype) {
             RankContext& c = e.context();
             const size_t bytes = static_cast<size_t>(numel_of(shape)) * c10::elementSize(dtype);
             const size_t off = c.arena_alloc(bytes);
             return py::make_tuple(heap_tensor(c.heap().data(c.rank()) + off, shape, dtype, c.heap().device()),
                                   static_cast<int64_t>(off));
           })
      // Offset of a tensor inside this rank's symmetric data region, or -1 when it lives elsewhere.
      .def("heapOffset",
           [](Engine& e, const torch::Tensor& t) -> int64_t {
             RankContext& c = e.context();
             if (!t.is_cuda()) return -1;
             const auto* first = static_cast<const uint8_t*>(t.data_ptr());
             const uint8_t* base = c.heap().data(c.rank());
             const size_t span = c.heap().layout().data_bytes;
             if (first < base || first + t.nbytes() > base + span) return -1;
             return static_cast<int64_t>(first - base);
           })
      .def("arenaReset", [](Engine& e) { e.context().arena_reset(); })
      .def("peerTensor",
           [](Engine& e, int rank, int64_t heap_offset, const std::vector<int64_t>& shape, torch::ScalarType dtype) {
             RankContext& c = e.context();
             return heap_tensor(c.heap().data(rank) + heap_offset, shape, dtype, c.heap().device());
           });

  py::class_<LocalCluster>(m, "LocalCluster")
      .def(py::init<int, int, size_t>(), py::arg("world"), py::arg("device") = 0,
           py::arg("buffer_bytes") = size_t(64) << 20)
      .def("world", &LocalCluster::world)
      .def("regOp", &LocalCluster::regOp)
      .def("setTimeoutMs", &LocalCluster::set_timeout_ms)
      .def("setCtas", &LocalCluster::set_ctas)
      .def("setProtocolCheck", &LocalCluster::set_protocol_check)
      .def("setTrace", [](LocalCluster& c, bool on) { for (int r = 0; r < c.world(); ++r) c.context(r).set_trace(on); })
      .def("trace", [](LocalCluster& c, const std::string& name, int rank) { return trace_list(c.context(rank), name); })
      .def("reset", &LocalCluster::reset)
      .def("opInfo",
           [](LocalCluster& c, const std::string& name, int rank) {
             const RegisteredOp& op = c.context(rank).op(name);
             py::dict d;
             d["chains"] = op.lowered.chains.size();
             d["steps"] = op.lowered.steps.size();
             d["ctas"] = op.lowered.total_ctas;
             d["multicast"] = op.lowered.uses_multicast;
             return d;
           })
      .def("lastStatus",
           [](LocalCluster& c) {
             py::list out;
             for (const DeviceStatus& s : c.last_status()) {
               py::dict d;
               d["code"] = s.code; d["rank"] = s.rank; d["chain"] = s.chain; d["step"] = s.step;
               d["slot"] = s.slot; d["observed"] = s.observed; d["expected"] = s.expected;
               out.append(d);
             }
             return out;
           })
      .def("exeOp", [](LocalCluster& c, const std::string& name, const std::vector<torch::Tensor>& in,
                       std::vector<torch::Tensor>& out) {
        std::vector<const void*> ip; std::vector<size_t> ib; std::vector<void*> op; std::vector<size_t> ob;
        for (const auto& t : in) { check_tensor(t, "input"); ip.push_back(t.data_ptr()); ib.push_back(t.nbytes()); }
        for (auto& t : out) { check_tensor(t, "output"); op.push_back(t.data_ptr()); ob.push_back(t.nbytes()); }
        c.exeOp(name, ip, ib, op, ob, current_stream());
      });

  // OCS control-plane exchange over NVLink (see ocs/signal_board.h).  Records are lists of at most
  // 14 unsigned 32-bit words.  Each call returns (ok, missing_rank, host_us, records).
  py::class_<SignalBoard>(m, "OcsSignalBoard")
      .def(py::init([]() { return new SignalBoard(Engine::instance().context()); }))
      .def("all_gather",
           [](SignalBoard& b, const std::vector<uint32_t>& words, uint64_t timeout_us) {
             std::array<uint32_t, kBoardWords> mine{};
             TORCH_CHECK(words.size() <= kBoardWords, "a record holds at most ", kBoardWords, " words");
             std::copy(words.begin(), words.end(), mine.begin());
             std::vector<std::array<uint32_t, kBoardWords>> records;
             BoardStatus st;
             {
               py::gil_scoped_release release;
               st = b.all_gather(mine, &records, timeout_us);
             }
             py::list out;
             for (const auto& r : records) out.append(std::vector<uint32_t>(r.begin(), r.end()));
             return py::make_tuple(st.ok, st.missing_rank, st.host_us, out);
           },
           py::arg("words"), py::arg("timeout_us") = 1000000)
      .def("broadcast",
           [](SignalBoard& b, int root, const std::vector<uint32_t>& words, uint64_t timeout_us) {
             std::array<uint32_t, kBoardWords> record{};
             TORCH_CHECK(words.size() <= kBoardWords, "a record holds at most ", kBoardWords, " words");
             std::copy(words.begin(), words.end(), record.begin());
             BoardStatus st;
             {
               py::gil_scoped_release release;
               st = b.broadcast(root, &record, timeout_us);
             }
             return py::make_tuple(st.ok, st.missing_rank, st.host_us, std::vector<uint32_t>(record.begin(), record.end()));
           },
           py::arg("root"), py::arg("words"), py::arg("timeout_us") = 1000000)
      // Both rounds of a barrier in one launch: returns (ok, missing_rank, host_us, records, release).
      .def("gather_release",
           [](SignalBoard& b, int root, const std::vector<uint32_t>& words, const std::vector<uint32_t>& release,
              int compare_begin, int compare_end, uint64_t timeout_us) {
             std::array<uint32_t, kBoardWords> mine{}, rel{}, got{};
             TORCH_CHECK(words.size() <= kBoardWords && release.size() <= kBoardWords, "a record holds at most ",
                         kBoardWords, " words");
             std::copy(words.begin(), words.end(), mine.begin());
             std::copy(release.begin(), release.end(), rel.begin());
             std::vector<std::array<uint32_t, kBoardWords>> records;
             BoardStatus st;
             {
               py::gil_scoped_release unlock;
               st = b.gather_release(root, mine, rel, compare_begin, compare_end, &records, &got, timeout_us);
             }
             py::list out;
             for (const auto& r : records) out.append(std::vector<uint32_t>(r.begin(), r.end()));
             return py::make_tuple(st.ok, st.missing_rank, st.host_us, out, std::vector<uint32_t>(got.begin(), got.end()));
           },
           py::arg("root"), py::arg("words"), py::arg("release"), py::arg("compare_begin"), py::arg("compare_end"),
           py::arg("timeout_us") = 1000000)
      .def("barrier",
           [](SignalBoard& b, uint64_t timeout_us) {
             py::gil_scoped_release release;
             const BoardStatus st = b.barrier(timeout_us);
             return std::make_tuple(st.ok, st.missing_rank, st.host_us);
           },
           py::arg("timeout_us") = 1000000)
      .def("reset", &SignalBoard::reset)
      .def("rounds", &SignalBoard::rounds)
      .def("world", &SignalBoard::world);

  // Host-only helpers usable without a GPU (plan loader / validator / lowering).
  m.def("lower_plan_summary", [](const std::string& json_text, int rank, int world, int64_t buffer_bytes,
                                 uint32_t ctas, bool multicast) {
    Plan plan = load_plan(json_text);
    PlanLimits lim{rank, world, buffer_bytes / dtype_bytes(plan.dtype)};
    validate_plan(plan, lim);
    LowerOptions lo;
    lo.rank = rank; lo.world = world; lo.total_ctas = ctas; lo.multicast = multicast;
    LoweredProgram lp = lower_plan(plan, lo);
    py::dict d;
    d["chains"] = lp.chains.size();
    d["steps"] = lp.steps.size();
    d["ctas"] = lp.total_ctas;
    d["multicast"] = lp.uses_multicast;
    py::list chains;
    for (const Chain& c : lp.chains) {
      py::list steps;
      for (uint32_t k = 0; k < c.step_count; ++k) {
        const Step& s = lp.steps[c.step_begin + k];
        steps.append(py::make_tuple(static_cast<int>(s.kind), static_cast<int>(s.n_wait), static_cast<int>(s.n_notify),
                                    static_cast<int>(s.n_dep), s.peer, s.bytes, static_cast<int>(s.defer_barrier)));
      }
      py::dict cd;
      cd["ctas"] = c.num_ctas; cd["barriers"] = c.barriers_per_launch; cd["steps"] = steps;
      chains.append(cd);
    }
    d["chain_list"] = chains;
    return d;
  });

  // All ranks' plans together: abstract execution of the signal protocol (no GPU needed).
  m.def("check_world", [](const std::vector<std::string>& plans_json) {
    std::vector<Plan> plans;
    for (const std::string& text : plans_json) plans.push_back(load_plan(text));
    const WorldReport rep = check_world(plans);
    py::dict d;
    d["deadlock"] = rep.deadlock;
    d["detail"] = rep.detail;
    d["leftover_signals"] = rep.leftover_signals;
    d["misaligned_ops"] = rep.misaligned_ops;
    d["notifies"] = rep.notifies;
    d["waits"] = rep.waits;
    return d;
  });
  // Largest grid whose CTAs are all resident at once, and a request clamped to it.
  m.def("coresident_limit", &coresident_limit);
  m.def("clamp_coresident", &clamp_coresident);

  // Raises the engine's timeout error from host code (exercises the exception mapping without a GPU).
  m.def("_raise_timeout", [](const std::string& text) { throw TimeoutError(text); });

  auto common = m.def_submodule("common");
  py::class_<Environs>(common, "Environs")
      .def_static("listOpt", &Environs::list_options)
      .def_static("getEnv", [](const std::string& n) { return Environs::require(n); })
      .def_static("registerOpt", &Environs::register_option);

  bind_fused_ops(m);
  bind_rdma(m);
}
