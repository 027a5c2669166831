// All-to-all exchange of one file descriptor per rank between the processes of a node.
//
// The symmetric arena (csrc/comm/symm_arena.cu) exports each rank's physical allocation as a POSIX
// file descriptor; a descriptor only means something inside the process that owns it, so it has to
// travel as SCM_RIGHTS ancillary data over a Unix-domain socket.  Every rank listens on
// `<dir>/rank-<r>.sock`, a receiver thread accepts world-1 connections, and the calling thread
// connects to every peer and sends (rank, fd).  Every wait is bounded by `timeout_ms`.
//
// The reference has nothing comparable: its ranks are threads of one process and its "exchange" is a
// mutex-protected vector (rumus-distributed/src/collective.rs:16-79).
#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <poll.h>
#include <string>
#include <sys/socket.h>
#include <sys/un.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

using Clock = std::chrono::steady_clock;

int remaining_ms(Clock::time_point deadline) {
  auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count();
  return ms < 0 ? 0 : (int)ms;
}

bool make_addr(const std::string& path, sockaddr_un* a) {
  std::memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  if (path.size() + 1 > sizeof(a->sun_path)) return false;
  std::memcpy(a->sun_path, path.c_str(), path.size() + 1);
  return true;
}

int send_fd(int sock, int rank, int fd) {
  msghdr msg{};
  iovec iov{&rank, sizeof(rank)};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
  return sendmsg(sock, &msg, 0) == (ssize_t)sizeof(rank) ? 0 : -1;
}

int recv_fd(int sock, int* rank, int* fd) {
  msghdr msg{};
  iovec iov{rank, sizeof(*rank)};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  if (recvmsg(sock, &msg, 0) != (ssize_t)sizeof(*rank)) return -1;
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) return -1;
  std::memcpy(fd, CMSG_DATA(c), sizeof(int));
  return 0;
}

}  // namespace

extern "C" {

// out_fds[world]: out_fds[rank] = my_fd (not duplicated); the others are new descriptors owned by
// the caller.  Returns 0, or: 1 bad arguments, 2 socket setup failed, 3 timed out waiting for a
// peer, 4 a transfer failed.  On failure every descriptor received so far is closed.
int rb_fd_exchange(const char* dir, int rank, int world, int my_fd, int* out_fds, int timeout_ms) {
  if (!dir || world < 1 || rank < 0 || rank >= world || !out_fds) return 1;
  for (int r = 0; r < world; ++r) out_fds[r] = -1;
  out_fds[rank] = my_fd;
  if (world == 1) return 0;
  const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  const std::string base(dir);
  sockaddr_un me;
  if (!make_addr(base + "/rank-" + std::to_string(rank) + ".sock", &me)) return 1;
  const int lsock = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (lsock < 0) return 2;
  unlink(me.sun_path);
  if (bind(lsock, (sockaddr*)&me, sizeof(me)) != 0 || listen(lsock, world) != 0) {
    close(lsock);
    return 2;
  }
  int recv_status = 0;
  std::thread receiver([&] {
    for (int got = 0; got < world - 1; ++got) {
      pollfd p{lsock, POLLIN, 0};
      const int pr = poll(&p, 1, remaining_ms(deadline));
      if (pr <= 0) { recv_status = 3; return; }
      const int c = accept4(lsock, nullptr, nullptr, SOCK_CLOEXEC);
      if (c < 0) { recv_status = 4; return; }
      pollfd q{c, POLLIN, 0};
      int peer = -1, fd = -1;
      if (poll(&q, 1, remaining_ms(deadline)) <= 0 || recv_fd(c, &peer, &fd) != 0 || peer < 0 ||
          peer >= world || peer == rank || out_fds[peer] != -1) {
        if (fd >= 0) close(fd);
        close(c);
        recv_status = 4;
        return;
      }
      out_fds[peer] = fd;
      close(c);
    }
  });
  int send_status = 0;
  for (int k = 1; k < world && send_status == 0; ++k) {
    const int peer = (rank + k) % world;
    sockaddr_un to;
    if (!make_addr(base + "/rank-" + std::to_string(peer) + ".sock", &to)) { send_status = 1; break; }
    int s = -1;
    for (;;) {   // the peer may not be listening yet: retry until the deadline
      s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
      if (s < 0) { send_status = 2; break; }
      if (connect(s, (sockaddr*)&to, sizeof(to)) == 0) break;
      close(s);
      s = -1;
      if (remaining_ms(deadline) == 0) { send_status = 3; break; }
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    if (s < 0) break;
    if (send_fd(s, rank, my_fd) != 0) send_status = 4;
    close(s);
  }
  receiver.join();
  close(lsock);
  unlink(me.sun_path);
  const int status = send_status ? send_status : recv_status;
  if (status) {
    for (int r = 0; r < world; ++r)
      if (r != rank && out_fds[r] >= 0) { close(out_fds[r]); out_fds[r] = -1; }
  }
  return status;
}
}
