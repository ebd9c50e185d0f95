// Passing file descriptors between the ranks of one node.
//
// CUDA virtual-memory allocations and multicast objects are shared between
// processes as POSIX file descriptors, which can only travel over a UNIX-domain
// socket (SCM_RIGHTS).  Every rank runs a tiny server thread that hands out the
// descriptors it has published under a name; peers fetch them by (rank, name).
//
// Sockets live in the abstract namespace under "pccl/<job>/<rank>", where <job>
// identifies the launch (PCCL_JOB_ID, else MASTER_ADDR:MASTER_PORT, plus the
// uid), so concurrent jobs on a shared machine cannot collide and nothing is
// left behind in /tmp (the reference binds /tmp/pccl_{rank}.sock:
// csrc/common/socket_utils.cc:16-19, 115-154, 233-260).
#pragma once
#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <thread>

namespace pccl {

class FdServer {
 public:
  FdServer() = default;
  ~FdServer();
  FdServer(const FdServer&) = delete;
  FdServer& operator=(const FdServer&) = delete;

  // Start serving for `rank` of job `job`.  Idempotent.
  void start(const std::string& job, int rank);
  void stop();
  // Publish (or replace) a descriptor under `name`; the server keeps its own dup.
  void publish(const std::string& name, int fd);
  bool running() const { return running_.load(); }

  // Fetch descriptor `name` from `rank`'s server.  Retries until `timeout_ms`
  // elapsed (the peer may not have published yet).  Returns -1 on failure.
  static int fetch(const std::string& job, int rank, const std::string& name, int timeout_ms = 10000);
  static std::string default_job_id();

 private:
  void serve();
  int listen_fd_ = -1;
  int wake_fd_[2] = {-1, -1};
  std::thread thread_;
  std::atomic<bool> running_{false};
  std::mutex mutex_;
  std::map<std::string, int> fds_;
};

}  // namespace pccl
