// File-descriptor all-gather between the ranks of one node.
//
// Each rank listens on an abstract-namespace Unix socket named after the
// session, the tag and its rank; it connects to every peer and sends its
// descriptor as SCM_RIGHTS ancillary data together with a small header.  A
// helper thread accepts the world-1 incoming connections meanwhile, so no
// ordering between ranks is needed.  Every blocking step honours one overall
// deadline; a peer that never shows up makes the call return KB_ERR_TIMEOUT.
//
// This is the transport the symmetric heap uses for cuMem shareable handles
// and for the memfd segments of the CPU-only backend.  There is no counterpart
// in the reference, which moves all data through NCCL collectives
// (reference.py:91-119, gemm_rs/reference.py:59).
#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <string>
#include <thread>
#include <vector>

#include "../common/host_util.h"
#include "../include/kb200.h"

namespace {

struct Header {
  uint32_t magic;
  int32_t src_rank;
  int32_t has_fd;
};
constexpr uint32_t kMagic = 0x4b423230u;  // "KB20"

int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return static_cast<int64_t>(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

socklen_t make_addr(sockaddr_un* addr, const std::string& name) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  // Abstract namespace: first byte of sun_path is NUL, no filesystem entry.
  size_t n = name.size();
  if (n > sizeof(addr->sun_path) - 2) n = sizeof(addr->sun_path) - 2;
  memcpy(addr->sun_path + 1, name.data(), n);
  return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
}

std::string sock_name(const char* session, const char* tag, int rank) {
  return std::string("kb200/") + session + "/" + tag + "/" + std::to_string(rank);
}

bool send_msg(int sock, const Header& h, int fd) {
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec iov;
  iov.iov_base = const_cast<Header*>(&h);
  iov.iov_len = sizeof(h);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  if (fd >= 0) {
    memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  ssize_t n;
  do {
    n = sendmsg(sock, &msg, MSG_NOSIGNAL);
  } while (n < 0 && errno == EINTR);
  return n == static_cast<ssize_t>(sizeof(h));
}

bool recv_msg(int sock, Header* h, int* fd, int64_t deadline) {
  *fd = -1;
  for (;;) {
    const int64_t left = deadline - now_ms();
    if (left <= 0) return false;
    pollfd pfd = {sock, POLLIN, 0};
    const int pr = poll(&pfd, 1, static_cast<int>(left > 1000 ? 1000 : left));
    if (pr < 0 && errno != EINTR) return false;
    if (pr > 0) break;
  }
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec iov;
  iov.iov_base = h;
  iov.iov_len = sizeof(*h);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  ssize_t n;
  do {
    n = recvmsg(sock, &msg, MSG_CMSG_CLOEXEC);
  } while (n < 0 && errno == EINTR);
  if (n != static_cast<ssize_t>(sizeof(*h)) || h->magic != kMagic) return false;
  for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(fd, CMSG_DATA(c), sizeof(int));
  }
  return true;
}

// The other end of a connected Unix socket must run under this process's user:
// abstract socket names are visible to every process of the network namespace, so
// a foreign process could bind a rank's name first (and be sent a memory handle)
// or connect and hand in a descriptor of its own.
bool peer_is_same_user(int sock) {
  ucred cred;
  socklen_t len = sizeof(cred);
  if (getsockopt(sock, SOL_SOCKET, SO_PEERCRED, &cred, &len) != 0 || len != sizeof(cred)) return false;
  return cred.uid == geteuid();
}

}  // namespace

extern "C" int kb_fd_allgather(const char* session, const char* tag, int rank, int world, int my_fd, int* out_fds,
                               int timeout_ms) {
  if (session == nullptr || tag == nullptr || out_fds == nullptr || world < 1 || rank < 0 || rank >= world) {
    kb::set_error("kb_fd_allgather: bad arguments");
    return KB_ERR_ARG;
  }
  for (int i = 0; i < world; ++i) out_fds[i] = -1;
  out_fds[rank] = my_fd >= 0 ? fcntl(my_fd, F_DUPFD_CLOEXEC, 0) : -1;
  if (world == 1) return KB_OK;
  const int64_t deadline = now_ms() + (timeout_ms > 0 ? timeout_ms : 30000);

  const int lsock = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (lsock < 0) {
    kb::set_error("socket(): %s", strerror(errno));
    return KB_ERR_IO;
  }
  sockaddr_un addr;
  const socklen_t alen = make_addr(&addr, sock_name(session, tag, rank));
  if (bind(lsock, reinterpret_cast<sockaddr*>(&addr), alen) != 0 || listen(lsock, world) != 0) {
    kb::set_error("bind/listen on abstract socket failed: %s", strerror(errno));
    close(lsock);
    return KB_ERR_IO;
  }

  std::atomic<int> acc_status{KB_OK};
  std::vector<int> got(world, -1);
  std::vector<char> seen(world, 0);
  std::thread acceptor([&]() {
    int received = 0;
    while (received < world - 1) {
      const int64_t left = deadline - now_ms();
      if (left <= 0) {
        acc_status = KB_ERR_TIMEOUT;
        return;
      }
      pollfd pfd = {lsock, POLLIN, 0};
      const int pr = poll(&pfd, 1, static_cast<int>(left > 200 ? 200 : left));
      if (pr < 0 && errno != EINTR) {
        acc_status = KB_ERR_IO;
        return;
      }
      if (pr <= 0) continue;
      const int c = accept4(lsock, nullptr, nullptr, SOCK_CLOEXEC);
      if (c < 0) continue;
      if (!peer_is_same_user(c)) {
        close(c);
        continue;  // not one of this job's ranks
      }
      Header h;
      int fd = -1;
      const bool ok = recv_msg(c, &h, &fd, deadline);
      close(c);
      if (!ok || h.src_rank < 0 || h.src_rank >= world || h.src_rank == rank || seen[h.src_rank]) {
        if (fd >= 0) close(fd);
        continue;  // stray or duplicate connection: ignore, keep waiting
      }
      if ((h.has_fd != 0) != (fd >= 0)) {
        if (fd >= 0) close(fd);
        acc_status = KB_ERR_IO;
        return;
      }
      seen[h.src_rank] = 1;
      got[h.src_rank] = fd;
      ++received;
    }
  });

  int send_status = KB_OK;
  for (int step = 1; step < world && send_status == KB_OK; ++step) {
    const int peer = (rank + step) % world;
    sockaddr_un paddr;
    const socklen_t plen = make_addr(&paddr, sock_name(session, tag, peer));
    for (;;) {
      if (now_ms() >= deadline) {
        send_status = KB_ERR_TIMEOUT;
        break;
      }
      const int c = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
      if (c < 0) {
        send_status = KB_ERR_IO;
        break;
      }
      if (connect(c, reinterpret_cast<sockaddr*>(&paddr), plen) == 0) {
        if (!peer_is_same_user(c)) {
          close(c);
          send_status = KB_ERR_IO;  // somebody else owns the peer's name: hand nothing over
          break;
        }
        Header h = {kMagic, rank, my_fd >= 0 ? 1 : 0};
        const bool ok = send_msg(c, h, my_fd);
        close(c);
        if (!ok) send_status = KB_ERR_IO;
        break;
      }
      close(c);
      usleep(2000);  // peer not listening yet
    }
  }
  acceptor.join();
  close(lsock);

  int rc = send_status != KB_OK ? send_status : acc_status.load();
  if (rc != KB_OK) {
    for (int i = 0; i < world; ++i) {
      if (got[i] >= 0) close(got[i]);
    }
    if (out_fds[rank] >= 0) {
      close(out_fds[rank]);
      out_fds[rank] = -1;
    }
    kb::set_error("kb_fd_allgather(%s/%s) rank %d: %s", session, tag, rank,
                  rc == KB_ERR_TIMEOUT ? "timed out waiting for peers" : "socket error");
    return rc;
  }
  for (int i = 0; i < world; ++i) {
    if (i != rank) out_fds[i] = got[i];
  }
  return KB_OK;
}
