// Loopback fabric and proxy thread of the RDMA executor (see rdma_transport.h).
#include <chrono>
#include <cstring>

#include "../../common/json.h"
#include "../../common/util.h"
#include "rdma_transport.h"

namespace pccl {
namespace rdma {

const char* status_name(Status s) {
  switch (s) {
    case Status::kOk: return "ok";
    case Status::kPending: return "pending";
    case Status::kTimeout: return "timeout";
    case Status::kRemoteAccessError: return "remote_access_error";
    case Status::kTransportError: return "transport_error";
    case Status::kNotConnected: return "not_connected";
    case Status::kShutdown: return "shutdown";
  }
  return "unknown";
}

std::string ConnectionInfo::to_json() const {
  json::Value v = json::Value::object();
  v.set("lid", static_cast<int64_t>(lid));
  v.set("gid", to_hex(gid, sizeof gid));
  v.set("qp_num", static_cast<int64_t>(qp_num));
  v.set("psn", static_cast<int64_t>(psn));
  return v.dump();
}

ConnectionInfo ConnectionInfo::from_json(const std::string& text) {
  const json::Value v = json::parse(text);
  ConnectionInfo c;
  c.lid = static_cast<uint16_t>(v.at("lid").as_int());
  const std::vector<uint8_t> raw = from_hex(v.at("gid").as_string());
  PCCL_CHECK(raw.size() == sizeof c.gid, "RDMA connection info: gid must be 16 bytes");
  std::memcpy(c.gid, raw.data(), sizeof c.gid);
  c.qp_num = static_cast<uint32_t>(v.at("qp_num").as_int());
  c.psn = static_cast<uint32_t>(v.at("psn").as_int());
  return c;
}

// ---- loopback fabric ---------------------------------------------------------------------------------------
class LoopbackFabric {
 public:
  explicit LoopbackFabric(int world) : ranks(world) {}
  struct Region { uint64_t addr, size; uint32_t rkey; };
  struct Pending { uint64_t wr_id; Status status; std::chrono::steady_clock::time_point ready; };
  struct Rank {
    std::vector<Region> regions;
    std::unordered_map<int, uint32_t> qp_of_peer;       // queue pairs this rank prepared
    std::unordered_map<int, MemoryKey> remote_of_peer;  // connected peers
    std::deque<Pending> pending;
    int fail_count = 0;
    Status fail_status = Status::kTransportError;
    int delay_us = 0;
    bool drop = false;
  };
  std::mutex mu;
  std::vector<Rank> ranks;
  uint32_t next_key = 0x1000, next_qp = 100;
};

std::shared_ptr<LoopbackFabric> make_loopback_fabric(int world) { return std::make_shared<LoopbackFabric>(world); }

void loopback_fail_next(LoopbackFabric& f, int rank, int count, Status status) {
  std::lock_guard<std::mutex> lock(f.mu);
  f.ranks.at(rank).fail_count = count;
  f.ranks.at(rank).fail_status = status;
}
void loopback_set_delay(LoopbackFabric& f, int rank, int micros) {
  std::lock_guard<std::mutex> lock(f.mu);
  f.ranks.at(rank).delay_us = micros;
}
void loopback_set_drop(LoopbackFabric& f, int rank, bool on) {
  std::lock_guard<std::mutex> lock(f.mu);
  f.ranks.at(rank).drop = on;
}

namespace {

class LoopbackTransport final : public Transport {
 public:
  LoopbackTransport(std::shared_ptr<LoopbackFabric> fabric, int rank) : fabric_(std::move(fabric)), rank_(rank) {}
  std::string name() const override { return "loopback"; }

  MemoryKey register_memory(void* addr, uint64_t size) override {
    std::lock_guard<std::mutex> lock(fabric_->mu);
    MemoryKey key;
    key.addr = reinterpret_cast<uint64_t>(addr);
    key.size = size;
    key.lkey = fabric_->next_key++;
    key.rkey = fabric_->next_key++;
    fabric_->ranks.at(rank_).regions.push_back({key.addr, size, key.rkey});
    return key;
  }
  void deregister_memory(const MemoryKey& key) override {
    std::lock_guard<std::mutex> lock(fabric_->mu);
    auto& regions = fabric_->ranks.at(rank_).regions;
    for (size_t i = 0; i < regions.size(); ++i)
      if (regions[i].rkey == key.rkey) { regions.erase(regions.begin() + i); break; }
  }
  ConnectionInfo prepare(int peer) override {
    std::lock_guard<std::mutex> lock(fabric_->mu);
    ConnectionInfo info;
    info.lid = static_cast<uint16_t>(rank_ + 1);
    info.gid[15] = static_cast<uint8_t>(rank_);
    info.qp_num = fabric_->next_qp++;
    fabric_->ranks.at(rank_).qp_of_peer[peer] = info.qp_num;
    return info;
  }
  Status connect(int peer, const ConnectionInfo& remote, const MemoryKey& remote_memory) override {
    std::lock_guard<std::mutex> lock(fabric_->mu);
    if (peer < 0 || peer >= static_cast<int>(fabric_->ranks.size())) return Status::kNotConnected;
    auto& me = fabric_->ranks.at(rank_);
    if (!me.qp_of_peer.count(peer)) return Status::kNotConnected;            // prepare() first
    // The queue-pair number must be the one the peer created for this rank.
    auto& other = fabric_->ranks.at(peer);
    auto it = other.qp_of_peer.find(rank_);
    if (it == other.qp_of_peer.end() || it->second != remote.qp_num) return Status::kNotConnected;
    me.remote_of_peer[peer] = remote_memory;
    return Status::kOk;
  }
  void disconnect(int peer) override {
    std::lock_guard<std::mutex> lock(fabric_->mu);
    fabric_->ranks.at(rank_).remote_of_peer.erase(peer);
  }
  Status post(Verb verb, int peer, const MemoryKey& local, uint64_t local_offset, uint64_t remote_offset,
              uint64_t size, uint64_t wr_id) override {
    std::lock_guard<std::mutex> lock(fabric_->mu);
    auto& me = fabric_->ranks.at(rank_);
    auto conn = me.remote_of_peer.find(peer);
    if (conn == me.remote_of_peer.end()) return Status::kNotConnected;
    if (me.drop) return Status::kOk;                                         // vanishes: never completes
    Status result = Status::kOk;
    if (me.fail_count > 0) {
      --me.fail_count;
      result = me.fail_status;
    } else {
      const MemoryKey& remote = conn->second;
      bool remote_ok = false;
      for (const auto& region : fabric_->ranks.at(peer).regions)
        if (region.rkey == remote.rkey && remote_offset + size <= region.size && region.addr == remote.addr)
          remote_ok = true;
      if (!remote_ok || local_offset + size > local.size) {
        result = Status::kRemoteAccessError;
      } else {
        uint8_t* mine = reinterpret_cast<uint8_t*>(local.addr) + local_offset;
        uint8_t* theirs = reinterpret_cast<uint8_t*>(remote.addr) + remote_offset;
        if (verb == Verb::kWrite) std::memcpy(theirs, mine, size);
        else std::memcpy(mine, theirs, size);
      }
    }
    me.pending.push_back({wr_id, result,
                          std::chrono::steady_clock::now() + std::chrono::microseconds(me.delay_us)});
    return Status::kOk;
  }
  int poll(Completion* out, int max) override {
    std::lock_guard<std::mutex> lock(fabric_->mu);
    auto& me = fabric_->ranks.at(rank_);
    const auto now = std::chrono::steady_clock::now();
    int n = 0;
    while (n < max && !me.pending.empty() && me.pending.front().ready <= now) {
      out[n].wr_id = me.pending.front().wr_id;
      out[n].status = me.pending.front().status;
      me.pending.pop_front();
      ++n;
    }
    return n;
  }

 private:
  std::shared_ptr<LoopbackFabric> fabric_;
  int rank_;
};

}  // namespace

std::unique_ptr<Transport> make_loopback_transport(std::shared_ptr<LoopbackFabric> fabric, int rank) {
  return std::make_unique<LoopbackTransport>(std::move(fabric), rank);
}

// ---- proxy --------------------------------------------------------------------------------------------------
Proxy::Proxy(std::unique_ptr<Transport> transport, void* local_base, uint64_t local_size)
    : transport_(std::move(transport)) {
  PCCL_CHECK(transport_ != nullptr, "RDMA proxy needs a transport (built without verbs?)");
  local_ = transport_->register_memory(local_base, local_size);
  worker_ = std::thread([this] { run(); });
}

Proxy::~Proxy() {
  stop();
  transport_->deregister_memory(local_);
}

void Proxy::stop() {
  {
    std::lock_guard<std::mutex> lock(mu_);
    if (stopping_) return;
    stopping_ = true;
  }
  cv_submit_.notify_all();
  cv_done_.notify_all();
  if (worker_.joinable()) worker_.join();
}

Status Proxy::connect(int peer, const ConnectionInfo& remote, const MemoryKey& remote_memory) {
  return transport_->connect(peer, remote, remote_memory);
}

int64_t Proxy::submit(const Command& cmd, int timeout_ms) {
  std::unique_lock<std::mutex> lock(mu_);
  const bool room = cv_done_.wait_for(lock, std::chrono::milliseconds(timeout_ms), [this] {
    return stopping_ || static_cast<int>(queue_.size()) + in_flight_ < kSlots;
  });
  if (!room || stopping_) return -1;
  const int64_t ticket = next_ticket_++;
  queue_.emplace_back(ticket, cmd);
  cv_submit_.notify_one();
  return ticket;
}

Status Proxy::wait(int64_t ticket, int timeout_ms) {
  std::unique_lock<std::mutex> lock(mu_);
  if (ticket < 0 || ticket >= next_ticket_) return Status::kNotConnected;
  const bool finished = cv_done_.wait_for(lock, std::chrono::milliseconds(timeout_ms),
                                          [&] { return stopping_ || done_.count(ticket) > 0; });
  auto it = done_.find(ticket);
  if (it != done_.end()) {
    const Status s = it->second;
    done_.erase(it);
    return s;
  }
  return finished && stopping_ ? Status::kShutdown : Status::kTimeout;
}

Status Proxy::drain(int timeout_ms) {
  std::unique_lock<std::mutex> lock(mu_);
  const bool idle = cv_done_.wait_for(lock, std::chrono::milliseconds(timeout_ms),
                                      [this] { return stopping_ || (queue_.empty() && in_flight_ == 0); });
  if (stopping_) return Status::kShutdown;
  if (!idle) return Status::kTimeout;
  Status worst = Status::kOk;
  for (const auto& kv : done_)
    if (kv.second != Status::kOk) worst = kv.second;
  done_.clear();
  return worst;
}

void Proxy::run() {
  std::vector<Completion> batch(32);
  while (true) {
    std::pair<int64_t, Command> next;
    bool have = false;
    {
      std::unique_lock<std::mutex> lock(mu_);
      if (queue_.empty() && in_flight_ == 0)
        cv_submit_.wait(lock, [this] { return stopping_ || !queue_.empty(); });
      if (stopping_) return;
      if (!queue_.empty()) {
        next = queue_.front();
        queue_.pop_front();
        ++in_flight_;
        have = true;
      }
    }
    if (have) {
      const Command& c = next.second;
      const Status posted = transport_->post(c.verb, c.peer, local_, c.local_offset, c.remote_offset, c.size,
                                             static_cast<uint64_t>(next.first));
      if (posted != Status::kOk) {
        std::lock_guard<std::mutex> lock(mu_);
        done_[next.first] = posted;
        --in_flight_;
        completed_.fetch_add(1);
        cv_done_.notify_all();
      }
    }
    const int n = transport_->poll(batch.data(), static_cast<int>(batch.size()));
    if (n > 0) {
      std::lock_guard<std::mutex> lock(mu_);
      for (int i = 0; i < n; ++i) {
        done_[static_cast<int64_t>(batch[i].wr_id)] = batch[i].status;
        --in_flight_;
        completed_.fetch_add(1);
      }
      cv_done_.notify_all();
    } else if (!have) {
      std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
  }
}

}  // namespace rdma
}  // namespace pccl
