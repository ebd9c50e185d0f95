// RDMA executor: transport interface, the in-process loopback fabric used by the unit tests,
// and the proxy thread that turns `rdma.write` / `rdma.read` commands into posted work requests.
//
// Inside one NVSwitch domain `rdma.*` plan operations are lowered to NVLink peer stores / loads
// (every peer's heap is mapped), so this path is only taken for peers that are not mapped, i.e.
// other nodes.  It is host-driven: the engine enqueues commands at stream-ordered points and no
// GPU thread ever spins on host memory.  The verbs transport is compiled only with
// PCCL_RDMA_ENABLED (needs <infiniband/verbs.h>); everything else builds without it.
//
// Reference counterparts: csrc/plugins/host/host_device.cc:182-430 (verbs set-up, RC queue
// pairs, memory registration) and csrc/plugins/host/host_proxy.{h,cc} (command queue + poll
// thread).  Unlike there, the queue-pair handshake is complete (INIT -> RTR -> RTS with the
// peer's queue-pair number from a second exchange) and every wait is bounded.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

namespace pccl {
namespace rdma {

enum class Status : int32_t {
  kOk = 0,
  kPending = 1,
  kTimeout = 2,
  kRemoteAccessError = 3,   // bad rkey / out-of-range remote address
  kTransportError = 4,      // queue pair in error state, flushed request, injected fault
  kNotConnected = 5,
  kShutdown = 6,
};
const char* status_name(Status s);

struct MemoryKey {          // what a peer needs to address registered memory
  uint64_t addr = 0, size = 0;
  uint32_t lkey = 0, rkey = 0;
};

struct ConnectionInfo {     // exchanged through the engine's endpoint JSON
  uint16_t lid = 0;
  uint8_t gid[16] = {};
  uint32_t qp_num = 0;      // queue pair this rank created for the receiving peer
  uint32_t psn = 0;
  std::string to_json() const;
  static ConnectionInfo from_json(const std::string& text);
};

struct Completion {
  uint64_t wr_id = 0;
  Status status = Status::kOk;
};

enum class Verb : int32_t { kWrite = 1, kRead = 2 };

class Transport {
 public:
  virtual ~Transport() = default;
  virtual std::string name() const = 0;
  // Register [addr, addr + size) for local and remote access.
  virtual MemoryKey register_memory(void* addr, uint64_t size) = 0;
  virtual void deregister_memory(const MemoryKey& key) = 0;
  // Create the queue pair towards `peer` (state INIT) and say how the peer can reach it.
  virtual ConnectionInfo prepare(int peer) = 0;
  // Second half of the handshake: the peer's ConnectionInfo and registered memory -> RTR -> RTS.
  virtual Status connect(int peer, const ConnectionInfo& remote, const MemoryKey& remote_memory) = 0;
  virtual void disconnect(int peer) = 0;
  // One-sided transfer between offsets of the local and the peer's registered memory.
  virtual Status post(Verb verb, int peer, const MemoryKey& local, uint64_t local_offset, uint64_t remote_offset,
                      uint64_t size, uint64_t wr_id) = 0;
  // Up to `max` finished requests; never blocks.
  virtual int poll(Completion* out, int max) = 0;
};

// ---- loopback fabric: N ranks inside one process, transfers are memcpy, faults can be injected ----
class LoopbackFabric;
std::shared_ptr<LoopbackFabric> make_loopback_fabric(int world);
std::unique_ptr<Transport> make_loopback_transport(std::shared_ptr<LoopbackFabric> fabric, int rank);
// Fault injection (tests): the next `count` posts from `rank` complete with `status` instead of moving data.
void loopback_fail_next(LoopbackFabric& fabric, int rank, int count, Status status);
// Every post from `rank` is held back for `micros` before it completes.
void loopback_set_delay(LoopbackFabric& fabric, int rank, int micros);
// Requests from `rank` are silently dropped (never complete) while `on`.
void loopback_set_drop(LoopbackFabric& fabric, int rank, bool on);

// Verbs transport over the first InfiniBand / RoCE device; null when compiled without verbs.
std::unique_ptr<Transport> make_verbs_transport(int port = 1, int gid_index = 0);
bool verbs_compiled();

// ---- proxy: command queue + worker thread ------------------------------------------------------------------
struct Command {
  Verb verb;
  int peer;
  uint64_t local_offset, remote_offset, size;
};

class Proxy {
 public:
  static constexpr int kSlots = 256;            // outstanding commands (reference: PROXY_QUEUE_CAPACITY)
  Proxy(std::unique_ptr<Transport> transport, void* local_base, uint64_t local_size);
  ~Proxy();
  Transport& transport() { return *transport_; }
  const MemoryKey& local_memory() const { return local_; }
  ConnectionInfo prepare(int peer) { return transport_->prepare(peer); }
  Status connect(int peer, const ConnectionInfo& remote, const MemoryKey& remote_memory);
  // Enqueue; returns a ticket, or -1 when all slots are busy for longer than timeout_ms.
  int64_t submit(const Command& cmd, int timeout_ms = 1000);
  // Wait (bounded) for a ticket; kTimeout leaves the command in flight.
  Status wait(int64_t ticket, int timeout_ms = 1000);
  // Wait for everything submitted so far.
  Status drain(int timeout_ms = 1000);
  uint64_t completed() const { return completed_.load(); }
  void stop();

 private:
  void run();
  std::unique_ptr<Transport> transport_;
  MemoryKey local_;
  std::mutex mu_;
  std::condition_variable cv_submit_, cv_done_;
  std::deque<std::pair<int64_t, Command>> queue_;
  std::unordered_map<int64_t, Status> done_;       // finished tickets not yet waited for
  int64_t next_ticket_ = 0;
  int in_flight_ = 0;
  std::atomic<uint64_t> completed_{0};
  bool stopping_ = false;
  std::thread worker_;
};

}  // namespace rdma
}  // namespace pccl
