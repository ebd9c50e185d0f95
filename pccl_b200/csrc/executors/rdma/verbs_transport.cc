// Verbs (InfiniBand / RoCE) transport of the RDMA executor.  Compiled to a stub unless
// PCCL_RDMA_ENABLED is defined (the build defines it when PCCL_RDMA=1 and
// <infiniband/verbs.h> is present).  One reliable-connected queue pair per peer, one
// completion queue, one registration per heap.
// Reference counterpart: csrc/plugins/host/host_device.cc:182-430.
#include "../../common/util.h"
#include "rdma_transport.h"

#ifdef PCCL_RDMA_ENABLED
#include <infiniband/verbs.h>

#include <cstring>
#include <random>
#endif

namespace pccl {
namespace rdma {

#ifndef PCCL_RDMA_ENABLED

std::unique_ptr<Transport> make_verbs_transport(int, int) { return nullptr; }
bool verbs_compiled() { return false; }

#else

namespace {

class VerbsTransport final : public Transport {
 public:
  VerbsTransport(int port, int gid_index) : port_(static_cast<uint8_t>(port)), gid_index_(gid_index) {
    int n = 0;
    ibv_device** list = ibv_get_device_list(&n);
    PCCL_CHECK(list && n > 0, "RDMA: no verbs device found");
    ctx_ = ibv_open_device(list[0]);
    ibv_free_device_list(list);
    PCCL_CHECK(ctx_, "RDMA: cannot open the verbs device");
    pd_ = ibv_alloc_pd(ctx_);
    PCCL_CHECK(pd_, "RDMA: cannot allocate a protection domain");
    cq_ = ibv_create_cq(ctx_, 4 * Proxy::kSlots, nullptr, nullptr, 0);
    PCCL_CHECK(cq_, "RDMA: cannot create the completion queue");
    ibv_port_attr attr{};
    PCCL_CHECK(ibv_query_port(ctx_, port_, &attr) == 0, "RDMA: cannot query port " << port);
    lid_ = attr.lid;
    mtu_ = attr.active_mtu;
    PCCL_CHECK(ibv_query_gid(ctx_, port_, gid_index_, &gid_) == 0, "RDMA: cannot query gid " << gid_index);
  }
  ~VerbsTransport() override {
    for (auto& kv : qps_) ibv_destroy_qp(kv.second.qp);
    for (auto& kv : mrs_) ibv_dereg_mr(kv.second);
    if (cq_) ibv_destroy_cq(cq_);
    if (pd_) ibv_dealloc_pd(pd_);
    if (ctx_) ibv_close_device(ctx_);
  }
  std::string name() const override { return "verbs"; }

  MemoryKey register_memory(void* addr, uint64_t size) override {
    ibv_mr* mr = ibv_reg_mr(pd_, addr, size,
                            IBV_ACCESS_LOCAL_WRITE | IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ);
    PCCL_CHECK(mr, "RDMA: ibv_reg_mr failed for " << size << " bytes");
    MemoryKey key;
    key.addr = reinterpret_cast<uint64_t>(addr);
    key.size = size;
    key.lkey = mr->lkey;
    key.rkey = mr->rkey;
    mrs_[key.rkey] = mr;
    return key;
  }
  void deregister_memory(const MemoryKey& key) override {
    auto it = mrs_.find(key.rkey);
    if (it == mrs_.end()) return;
    ibv_dereg_mr(it->second);
    mrs_.erase(it);
  }

  ConnectionInfo prepare(int peer) override {
    ibv_qp_init_attr init{};
    init.send_cq = cq_;
    init.recv_cq = cq_;
    init.qp_type = IBV_QPT_RC;
    init.cap.max_send_wr = Proxy::kSlots;
    init.cap.max_recv_wr = 1;
    init.cap.max_send_sge = 1;
    init.cap.max_recv_sge = 1;
    ibv_qp* qp = ibv_create_qp(pd_, &init);
    PCCL_CHECK(qp, "RDMA: cannot create the queue pair for peer " << peer);
    ibv_qp_attr attr{};
    attr.qp_state = IBV_QPS_INIT;
    attr.pkey_index = 0;
    attr.port_num = port_;
    attr.qp_access_flags = IBV_ACCESS_REMOTE_WRITE | IBV_ACCESS_REMOTE_READ;
    PCCL_CHECK(ibv_modify_qp(qp, &attr, IBV_QP_STATE | IBV_QP_PKEY_INDEX | IBV_QP_PORT | IBV_QP_ACCESS_FLAGS) == 0,
               "RDMA: queue pair for peer " << peer << " did not reach INIT");
    Peer p;
    p.qp = qp;
    p.psn = std::random_device{}() & 0xffffffu;
    qps_[peer] = p;
    ConnectionInfo info;
    info.lid = lid_;
    std::memcpy(info.gid, gid_.raw, sizeof info.gid);
    info.qp_num = qp->qp_num;
    info.psn = p.psn;
    return info;
  }

  Status connect(int peer, const ConnectionInfo& remote, const MemoryKey& remote_memory) override {
    auto it = qps_.find(peer);
    if (it == qps_.end()) return Status::kNotConnected;
    ibv_qp_attr attr{};
    attr.qp_state = IBV_QPS_RTR;
    attr.path_mtu = mtu_;
    attr.dest_qp_num = remote.qp_num;
    attr.rq_psn = remote.psn;
    attr.max_dest_rd_atomic = 16;
    attr.min_rnr_timer = 12;
    attr.ah_attr.dlid = remote.lid;
    attr.ah_attr.port_num = port_;
    attr.ah_attr.is_global = 1;
    std::memcpy(attr.ah_attr.grh.dgid.raw, remote.gid, 16);
    attr.ah_attr.grh.sgid_index = static_cast<uint8_t>(gid_index_);
    attr.ah_attr.grh.hop_limit = 64;
    if (ibv_modify_qp(it->second.qp, &attr,
                      IBV_QP_STATE | IBV_QP_AV | IBV_QP_PATH_MTU | IBV_QP_DEST_QPN | IBV_QP_RQ_PSN |
                          IBV_QP_MAX_DEST_RD_ATOMIC | IBV_QP_MIN_RNR_TIMER) != 0)
      return Status::kTransportError;
    std::memset(&attr, 0, sizeof attr);
    attr.qp_state = IBV_QPS_RTS;
    attr.timeout = 14;
    attr.retry_cnt = 7;
    attr.rnr_retry = 7;
    attr.sq_psn = it->second.psn;
    attr.max_rd_atomic = 16;
    if (ibv_modify_qp(it->second.qp, &attr,
                      IBV_QP_STATE | IBV_QP_TIMEOUT | IBV_QP_RETRY_CNT | IBV_QP_RNR_RETRY | IBV_QP_SQ_PSN |
                          IBV_QP_MAX_QP_RD_ATOMIC) != 0)
      return Status::kTransportError;
    it->second.remote = remote_memory;
    it->second.connected = true;
    return Status::kOk;
  }

  void disconnect(int peer) override {
    auto it = qps_.find(peer);
    if (it == qps_.end()) return;
    ibv_destroy_qp(it->second.qp);
    qps_.erase(it);
  }

  Status post(Verb verb, int peer, const MemoryKey& local, uint64_t local_offset, uint64_t remote_offset,
              uint64_t size, uint64_t wr_id) override {
    auto it = qps_.find(peer);
    if (it == qps_.end() || !it->second.connected) return Status::kNotConnected;
    const MemoryKey& remote = it->second.remote;
    if (local_offset + size > local.size || remote_offset + size > remote.size) return Status::kRemoteAccessError;
    ibv_sge sge{};
    sge.addr = local.addr + local_offset;
    sge.length = static_cast<uint32_t>(size);
    sge.lkey = local.lkey;
    ibv_send_wr wr{};
    wr.wr_id = wr_id;
    wr.sg_list = &sge;
    wr.num_sge = 1;
    wr.opcode = verb == Verb::kWrite ? IBV_WR_RDMA_WRITE : IBV_WR_RDMA_READ;
    wr.send_flags = IBV_SEND_SIGNALED;
    wr.wr.rdma.remote_addr = remote.addr + remote_offset;
    wr.wr.rdma.rkey = remote.rkey;
    ibv_send_wr* bad = nullptr;
    return ibv_post_send(it->second.qp, &wr, &bad) == 0 ? Status::kOk : Status::kTransportError;
  }

  int poll(Completion* out, int max) override {
    ibv_wc wc[32];
    const int n = ibv_poll_cq(cq_, max < 32 ? max : 32, wc);
    for (int i = 0; i < n; ++i) {
      out[i].wr_id = wc[i].wr_id;
      out[i].status = wc[i].status == IBV_WC_SUCCESS
                          ? Status::kOk
                          : (wc[i].status == IBV_WC_REM_ACCESS_ERR ? Status::kRemoteAccessError
                                                                   : Status::kTransportError);
    }
    return n < 0 ? 0 : n;
  }

 private:
  struct Peer {
    ibv_qp* qp = nullptr;
    uint32_t psn = 0;
    MemoryKey remote;
    bool connected = false;
  };
  uint8_t port_;
  int gid_index_;
  ibv_context* ctx_ = nullptr;
  ibv_pd* pd_ = nullptr;
  ibv_cq* cq_ = nullptr;
  uint16_t lid_ = 0;
  ibv_mtu mtu_ = IBV_MTU_1024;
  ibv_gid gid_{};
  std::unordered_map<int, Peer> qps_;
  std::unordered_map<uint32_t, ibv_mr*> mrs_;
};

}  // namespace

std::unique_ptr<Transport> make_verbs_transport(int port, int gid_index) {
  return std::make_unique<VerbsTransport>(port, gid_index);
}
bool verbs_compiled() { return true; }

#endif  // PCCL_RDMA_ENABLED

}  // namespace rdma
}  // namespace pccl
