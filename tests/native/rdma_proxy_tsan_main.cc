// The RDMA proxy (command queue + worker thread) over the in-process loopback fabric, under
// ThreadSanitizer: two ranks, several submitting threads per rank, writes and reads to disjoint
// ranges, an injected transport error, dropped requests that must time out, and shutdown with
// commands still queued.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <memory>
#include <thread>
#include <vector>

#include "executors/rdma/rdma_transport.h"

using namespace pccl::rdma;

int main() {
  constexpr uint64_t kBytes = 1 << 20, kChunk = 4096;
  constexpr int kThreads = 4, kPerThread = 32;
  auto fabric = make_loopback_fabric(2);
  std::vector<std::vector<uint8_t>> memory(2, std::vector<uint8_t>(kBytes));
  for (int r = 0; r < 2; ++r)
    for (uint64_t i = 0; i < kBytes; ++i) memory[r][i] = static_cast<uint8_t>((i * 7 + r * 13) & 0xff);
  const std::vector<std::vector<uint8_t>> original = memory;
  std::vector<std::unique_ptr<Proxy>> proxy;
  for (int r = 0; r < 2; ++r)
    proxy.push_back(std::make_unique<Proxy>(make_loopback_transport(fabric, r), memory[r].data(), kBytes));
  std::atomic<int> failures{0};
  ConnectionInfo info[2] = {proxy[0]->prepare(1), proxy[1]->prepare(0)};
  if (proxy[0]->connect(1, info[1], proxy[1]->local_memory()) != Status::kOk) ++failures;
  if (proxy[1]->connect(0, info[0], proxy[0]->local_memory()) != Status::kOk) ++failures;

  // Rank 0 writes the first half of its memory into the peer's second half; rank 1 reads the peer's
  // second half... no: ranges are chosen so that no byte is both read and written (the data race
  // would be the test's own): rank 0 writes [0, 512K) -> peer [512K, 1M); rank 1 reads peer
  // [512K, 1M) -> own [0, 512K).  Every thread owns a disjoint set of chunks.
  std::vector<std::thread> threads;
  for (int r = 0; r < 2; ++r) {
    for (int t = 0; t < kThreads; ++t) {
      threads.emplace_back([&, r, t] {
        std::vector<int64_t> tickets;
        for (int i = 0; i < kPerThread; ++i) {
          const uint64_t chunk = static_cast<uint64_t>(t * kPerThread + i);
          Command cmd{r == 0 ? Verb::kWrite : Verb::kRead, 1 - r, chunk * kChunk, kBytes / 2 + chunk * kChunk, kChunk};
          const int64_t ticket = proxy[r]->submit(cmd, 2000);
          if (ticket < 0) { ++failures; continue; }
          tickets.push_back(ticket);
        }
        for (const int64_t ticket : tickets)
          if (proxy[r]->wait(ticket, 5000) != Status::kOk) ++failures;
      });
    }
  }
  for (auto& t : threads) t.join();
  const uint64_t moved = static_cast<uint64_t>(kThreads) * kPerThread * kChunk;
  if (std::memcmp(memory[1].data() + kBytes / 2, original[0].data(), moved) != 0) ++failures;   // rank 0's writes
  if (std::memcmp(memory[1].data(), original[0].data() + kBytes / 2, moved) != 0) ++failures;   // rank 1's reads

  // injected transport error, reported on the ticket
  loopback_fail_next(*fabric, 0, 1, Status::kTransportError);
  int64_t ticket = proxy[0]->submit(Command{Verb::kWrite, 1, 0, 0, 64}, 1000);
  if (ticket < 0 || proxy[0]->wait(ticket, 2000) != Status::kTransportError) ++failures;
  // out of range: refused by the fabric
  ticket = proxy[0]->submit(Command{Verb::kWrite, 1, 0, kBytes - 8, 64}, 1000);
  if (ticket < 0 || proxy[0]->wait(ticket, 2000) == Status::kOk) ++failures;
  // dropped requests: the wait runs out, the proxy stays usable afterwards
  loopback_set_drop(*fabric, 1, true);
  ticket = proxy[1]->submit(Command{Verb::kRead, 0, 0, 0, 64}, 1000);
  if (ticket < 0 || proxy[1]->wait(ticket, 200) != Status::kTimeout) ++failures;
  loopback_set_drop(*fabric, 1, false);
  ticket = proxy[1]->submit(Command{Verb::kRead, 0, 0, 0, 64}, 1000);
  if (ticket < 0 || proxy[1]->wait(ticket, 2000) != Status::kOk) ++failures;

  // shutdown with work queued behind a delay
  loopback_set_delay(*fabric, 0, 2000);
  for (int i = 0; i < 16; ++i) proxy[0]->submit(Command{Verb::kWrite, 1, 0, 0, 64}, 1000);
  proxy[0]->stop();
  proxy[1]->stop();
  proxy.clear();
  std::printf("RDMA_PROXY_TSAN failures=%d\n", failures.load());
  return failures.load() == 0 ? 0 : 1;
}
