#include "fd_socket.h"

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <chrono>
#include <cstring>

#include "util.h"

namespace pccl {
namespace {

constexpr char kMagic[] = "PCCLFD1";

socklen_t make_address(const std::string& job, int rank, sockaddr_un* addr) {
  std::memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  const std::string name = "pccl/" + job + "/" + std::to_string(rank);
  const size_t n = std::min(name.size(), sizeof(addr->sun_path) - 2);
  // Leading NUL byte selects the abstract namespace.
  std::memcpy(addr->sun_path + 1, name.data(), n);
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

bool send_fd(int sock, int fd) {
  char payload = fd >= 0 ? 'Y' : 'N';
  iovec iov{&payload, 1};
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  if (fd >= 0) {
    std::memset(control, 0, sizeof control);
    msg.msg_control = control;
    msg.msg_controllen = sizeof control;
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  return sendmsg(sock, &msg, MSG_NOSIGNAL) == 1;
}

int recv_fd(int sock) {
  char payload = 0;
  iovec iov{&payload, 1};
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char control[CMSG_SPACE(sizeof(int))];
  msg.msg_control = control;
  msg.msg_controllen = sizeof control;
  if (recvmsg(sock, &msg, 0) != 1 || payload != 'Y') return -1;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
      int fd = -1;
      std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
      return fd;
    }
  }
  return -1;
}

void set_timeouts(int sock, int ms) {
  timeval tv{ms / 1000, (ms % 1000) * 1000};
  setsockopt(sock, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
  setsockopt(sock, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
}

}  // namespace

std::string FdServer::default_job_id() {
  std::string job = Environs::get("PCCL_JOB_ID");
  if (job.empty()) {
    const std::string port = Environs::get("MASTER_PORT");
    job = port.empty() ? "local" : Environs::get("MASTER_ADDR", "localhost") + ":" + port;
  }
  return job + "/u" + std::to_string(static_cast<long>(getuid()));
}

FdServer::~FdServer() { stop(); }

void FdServer::start(const std::string& job, int rank) {
  if (running_.load()) return;
  listen_fd_ = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  PCCL_CHECK(listen_fd_ >= 0, "fd server: socket() failed: " << std::strerror(errno));
  sockaddr_un addr;
  const socklen_t len = make_address(job, rank, &addr);
  if (bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), len) != 0 || listen(listen_fd_, 64) != 0) {
    const std::string why = std::strerror(errno);
    close(listen_fd_);
    listen_fd_ = -1;
    throw Error("fd server: cannot bind abstract socket for job '" + job + "' rank " +
                std::to_string(rank) + ": " + why);
  }
  PCCL_CHECK(pipe(wake_fd_) == 0, "fd server: pipe() failed");
  running_.store(true);
  thread_ = std::thread([this] { serve(); });
}

void FdServer::stop() {
  if (!running_.exchange(false)) return;
  char b = 1;
  (void)!write(wake_fd_[1], &b, 1);
  if (thread_.joinable()) thread_.join();
  close(listen_fd_);
  close(wake_fd_[0]);
  close(wake_fd_[1]);
  listen_fd_ = wake_fd_[0] = wake_fd_[1] = -1;
  std::lock_guard<std::mutex> lock(mutex_);
  for (auto& kv : fds_) close(kv.second);
  fds_.clear();
}

void FdServer::publish(const std::string& name, int fd) {
  const int copy = dup(fd);
  PCCL_CHECK(copy >= 0, "fd server: dup() failed: " << std::strerror(errno));
  std::lock_guard<std::mutex> lock(mutex_);
  auto it = fds_.find(name);
  if (it != fds_.end()) { close(it->second); it->second = copy; }
  else fds_[name] = copy;
}

void FdServer::serve() {
  while (running_.load()) {
    pollfd fds[2] = {{listen_fd_, POLLIN, 0}, {wake_fd_[0], POLLIN, 0}};
    if (poll(fds, 2, 500) <= 0) continue;
    if (fds[1].revents) break;
    if (!(fds[0].revents & POLLIN)) continue;
    const int conn = accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
    if (conn < 0) continue;
    // An abstract socket carries no file permissions, so the kernel-attested credentials of the
    // connecting process are the only authentication: descriptors of this job's heap go to
    // processes of the same user and to nobody else.
    ucred peer{};
    socklen_t peer_len = sizeof peer;
    if (getsockopt(conn, SOL_SOCKET, SO_PEERCRED, &peer, &peer_len) != 0 || peer.uid != getuid()) {
      PCCL_LOG_WARN("fd server: refused a connection from uid " << peer.uid << " (pid " << peer.pid << ")");
      close(conn);
      continue;
    }
    set_timeouts(conn, 2000);
    // Request: magic, one length byte, name.
    char head[sizeof(kMagic) + 1];
    bool ok = recv(conn, head, sizeof head, MSG_WAITALL) == static_cast<ssize_t>(sizeof head) &&
              std::memcmp(head, kMagic, sizeof(kMagic)) == 0;
    std::string name;
    if (ok) {
      name.resize(static_cast<unsigned char>(head[sizeof(kMagic)]));
      ok = name.empty() || recv(conn, &name[0], name.size(), MSG_WAITALL) == static_cast<ssize_t>(name.size());
    }
    int fd = -1;
    if (ok) {
      std::lock_guard<std::mutex> lock(mutex_);
      auto it = fds_.find(name);
      if (it != fds_.end()) fd = it->second;
    }
    send_fd(conn, fd);
    close(conn);
  }
}

int FdServer::fetch(const std::string& job, int rank, const std::string& name, int timeout_ms) {
  PCCL_CHECK(name.size() < 256, "fd name too long");
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  sockaddr_un addr;
  const socklen_t len = make_address(job, rank, &addr);
  do {
    const int sock = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (sock < 0) return -1;
    set_timeouts(sock, 2000);
    if (connect(sock, reinterpret_cast<sockaddr*>(&addr), len) == 0) {
      std::string req(kMagic, sizeof(kMagic));
      req.push_back(static_cast<char>(name.size()));
      req += name;
      if (send(sock, req.data(), req.size(), MSG_NOSIGNAL) == static_cast<ssize_t>(req.size())) {
        const int fd = recv_fd(sock);
        close(sock);
        if (fd >= 0) return fd;
      } else {
        close(sock);
      }
    } else {
      close(sock);
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  } while (std::chrono::steady_clock::now() < deadline);
  return -1;
}

}  // namespace pccl
