// The descriptor server under ThreadSanitizer: several servers (one per "rank"), concurrent
// publishers and fetchers, replacement of a published descriptor, a fetch of a name nobody
// publishes (must time out, not hang), stop while clients are still connecting.
// Every fetched descriptor must read back the bytes that were written through the original.
#include <fcntl.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "common/fd_socket.h"

namespace {

int make_file(const std::string& text) {
  char path[] = "/tmp/pccl_fd_test_XXXXXX";
  const int fd = mkstemp(path);
  if (fd < 0) return -1;
  unlink(path);
  if (write(fd, text.data(), text.size()) != static_cast<ssize_t>(text.size())) return -1;
  return fd;
}

std::string read_all(int fd) {
  char buf[256];
  const ssize_t n = pread(fd, buf, sizeof buf, 0);
  return n > 0 ? std::string(buf, static_cast<size_t>(n)) : std::string();
}

}  // namespace

int main() {
  const std::string job = "tsan-" + std::to_string(getpid());
  constexpr int kRanks = 4, kNames = 3;
  std::vector<pccl::FdServer> servers(kRanks);
  for (int r = 0; r < kRanks; ++r) servers[r].start(job, r);
  std::atomic<int> failures{0};

  // publishers race with fetchers: a fetch retries until the name appears
  std::vector<std::thread> threads;
  for (int r = 0; r < kRanks; ++r) {
    threads.emplace_back([&, r] {
      for (int n = 0; n < kNames; ++n) {
        const std::string text = "rank" + std::to_string(r) + "-name" + std::to_string(n);
        const int fd = make_file(text);
        if (fd < 0) { ++failures; continue; }
        servers[r].publish("obj" + std::to_string(n), fd);
        close(fd);                                   // the server keeps its own duplicate
      }
    });
  }
  for (int client = 0; client < kRanks; ++client) {
    threads.emplace_back([&, client] {
      for (int r = 0; r < kRanks; ++r) {
        for (int n = 0; n < kNames; ++n) {
          const int fd = pccl::FdServer::fetch(job, r, "obj" + std::to_string(n), 5000);
          const std::string want = "rank" + std::to_string(r) + "-name" + std::to_string(n);
          if (fd < 0 || read_all(fd) != want) {
            std::fprintf(stderr, "client %d: rank %d obj%d mismatch\n", client, r, n);
            ++failures;
          }
          if (fd >= 0) close(fd);
        }
      }
    });
  }
  for (auto& t : threads) t.join();
  threads.clear();

  // replacing a descriptor serves the new one
  const int newer = make_file("replaced");
  servers[0].publish("obj0", newer);
  close(newer);
  const int got = pccl::FdServer::fetch(job, 0, "obj0", 2000);
  if (got < 0 || read_all(got) != "replaced") ++failures;
  if (got >= 0) close(got);

  // a name nobody publishes: bounded failure
  if (pccl::FdServer::fetch(job, 1, "missing", 300) != -1) ++failures;
  // a rank nobody serves: bounded failure
  if (pccl::FdServer::fetch(job, 17, "obj0", 300) != -1) ++failures;

  // stop while clients keep asking
  std::thread asker([&] {
    for (int i = 0; i < 50; ++i) {
      const int fd = pccl::FdServer::fetch(job, 2, "obj1", 50);
      if (fd >= 0) close(fd);
    }
  });
  servers[2].stop();
  asker.join();
  for (auto& s : servers) s.stop();
  std::printf("FD_SERVER_TSAN failures=%d\n", failures.load());
  return failures.load() == 0 ? 0 : 1;
}
