// Python bindings of the RDMA executor: fabric, proxy and fault injection for the unit tests.
#include <torch/extension.h>

#include "../../common/util.h"
#include "rdma_transport.h"

namespace py = pybind11;

namespace pccl {

namespace {

// The fabric type is opaque outside its translation unit: hand Python a holder.
struct FabricHandle {
  std::shared_ptr<rdma::LoopbackFabric> fabric;
};

// A proxy bound to a CPU byte tensor that stands for the registered heap.
struct BoundProxy {
  torch::Tensor memory;
  std::unique_ptr<rdma::Proxy> proxy;
};

}  // namespace

void bind_rdma(py::module_& m) {
  auto r = m.def_submodule("rdma", "RDMA executor: transports, proxy thread, loopback fabric");
  r.def("verbs_compiled", &rdma::verbs_compiled);
  py::enum_<rdma::Status>(r, "Status")
      .value("OK", rdma::Status::kOk)
      .value("PENDING", rdma::Status::kPending)
      .value("TIMEOUT", rdma::Status::kTimeout)
      .value("REMOTE_ACCESS_ERROR", rdma::Status::kRemoteAccessError)
      .value("TRANSPORT_ERROR", rdma::Status::kTransportError)
      .value("NOT_CONNECTED", rdma::Status::kNotConnected)
      .value("SHUTDOWN", rdma::Status::kShutdown);
  r.def("status_name", &rdma::status_name);

  py::class_<FabricHandle>(r, "LoopbackFabric")
      .def(py::init([](int world) { return FabricHandle{rdma::make_loopback_fabric(world)}; }), py::arg("world"))
      .def("fail_next", [](FabricHandle& f, int rank, int count, rdma::Status s) {
        rdma::loopback_fail_next(*f.fabric, rank, count, s);
      }, py::arg("rank"), py::arg("count"), py::arg("status") = rdma::Status::kTransportError)
      .def("set_delay_us", [](FabricHandle& f, int rank, int us) { rdma::loopback_set_delay(*f.fabric, rank, us); })
      .def("set_drop", [](FabricHandle& f, int rank, bool on) { rdma::loopback_set_drop(*f.fabric, rank, on); });

  py::class_<BoundProxy>(r, "Proxy")
      .def(py::init([](FabricHandle& fabric, int rank, torch::Tensor memory) {
             TORCH_CHECK(!memory.is_cuda() && memory.is_contiguous(), "loopback memory must be a contiguous CPU tensor");
             auto bound = std::make_unique<BoundProxy>();
             bound->memory = memory;
             bound->proxy = std::make_unique<rdma::Proxy>(rdma::make_loopback_transport(fabric.fabric, rank),
                                                          memory.data_ptr(), memory.nbytes());
             return bound;
           }),
           py::arg("fabric"), py::arg("rank"), py::arg("memory"))
      // Endpoint fragment this rank publishes for `peer`: connection info + registered memory.
      .def("prepare", [](BoundProxy& b, int peer) {
        const rdma::ConnectionInfo info = b.proxy->prepare(peer);
        const rdma::MemoryKey& k = b.proxy->local_memory();
        py::dict d;
        d["conn"] = info.to_json();
        d["addr"] = k.addr;
        d["size"] = k.size;
        d["rkey"] = k.rkey;
        return d;
      })
      .def("connect", [](BoundProxy& b, int peer, const py::dict& remote) {
        rdma::MemoryKey k;
        k.addr = remote["addr"].cast<uint64_t>();
        k.size = remote["size"].cast<uint64_t>();
        k.rkey = remote["rkey"].cast<uint32_t>();
        return b.proxy->connect(peer, rdma::ConnectionInfo::from_json(remote["conn"].cast<std::string>()), k);
      })
      .def("write", [](BoundProxy& b, int peer, uint64_t local_off, uint64_t remote_off, uint64_t size, int timeout_ms) {
        return b.proxy->submit({rdma::Verb::kWrite, peer, local_off, remote_off, size}, timeout_ms);
      }, py::arg("peer"), py::arg("local_offset"), py::arg("remote_offset"), py::arg("size"),
         py::arg("timeout_ms") = 1000)
      .def("read", [](BoundProxy& b, int peer, uint64_t local_off, uint64_t remote_off, uint64_t size, int timeout_ms) {
        return b.proxy->submit({rdma::Verb::kRead, peer, local_off, remote_off, size}, timeout_ms);
      }, py::arg("peer"), py::arg("local_offset"), py::arg("remote_offset"), py::arg("size"),
         py::arg("timeout_ms") = 1000)
      .def("wait", [](BoundProxy& b, int64_t ticket, int timeout_ms) {
        py::gil_scoped_release release;
        return b.proxy->wait(ticket, timeout_ms);
      }, py::arg("ticket"), py::arg("timeout_ms") = 1000)
      .def("drain", [](BoundProxy& b, int timeout_ms) {
        py::gil_scoped_release release;
        return b.proxy->drain(timeout_ms);
      }, py::arg("timeout_ms") = 1000)
      .def("completed", [](BoundProxy& b) { return b.proxy->completed(); })
      .def("stop", [](BoundProxy& b) { b.proxy->stop(); });
}

}  // namespace pccl
