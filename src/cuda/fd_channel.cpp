#include "fd_channel.h"

#include <errno.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <thread>

#include "ibcomm/error.h"

namespace ibcomm {

std::string FdChannelName(unsigned pid, unsigned nonce) {
  char buf[64];
  snprintf(buf, sizeof(buf), "ibcomm.fd.%u.%08x", pid, nonce);
  return buf;
}

static socklen_t Fill(struct sockaddr_un* addr, const std::string& name) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  // Abstract namespace: leading NUL, no file system entry to clean up.
  size_t n = name.size() < sizeof(addr->sun_path) - 2 ? name.size() : sizeof(addr->sun_path) - 2;
  memcpy(addr->sun_path + 1, name.data(), n);
  return static_cast<socklen_t>(offsetof(struct sockaddr_un, sun_path) + 1 + n);
}

FdChannel::~FdChannel() {
  if (sock_ >= 0) close(sock_);
  if (listen_fd_ >= 0) close(listen_fd_);
}

void FdChannel::Listen(const std::string& name) {
  listen_fd_ = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (listen_fd_ < 0) IBCOMM_FAIL(TRANSPORT_ERROR, "socket() failed: %s\n", strerror(errno));
  struct sockaddr_un addr;
  socklen_t len = Fill(&addr, name);
  if (bind(listen_fd_, reinterpret_cast<struct sockaddr*>(&addr), len) != 0)
    IBCOMM_FAIL(TRANSPORT_ERROR, "bind(@%s) failed: %s\n", name.c_str(), strerror(errno));
  if (listen(listen_fd_, 4) != 0) IBCOMM_FAIL(TRANSPORT_ERROR, "listen(@%s) failed: %s\n", name.c_str(), strerror(errno));
}

void FdChannel::Accept(int timeout_ms) {
  struct pollfd p = {listen_fd_, POLLIN, 0};
  int rc = poll(&p, 1, timeout_ms);
  if (rc <= 0) IBCOMM_FAIL(TRANSPORT_ERROR, "No peer connected to the descriptor channel within %d ms.\n", timeout_ms);
  sock_ = accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
  if (sock_ < 0) IBCOMM_FAIL(TRANSPORT_ERROR, "accept() failed: %s\n", strerror(errno));
  close(listen_fd_);
  listen_fd_ = -1;
}

void FdChannel::Connect(const std::string& name, int timeout_ms) {
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (s < 0) IBCOMM_FAIL(TRANSPORT_ERROR, "socket() failed: %s\n", strerror(errno));
    struct sockaddr_un addr;
    socklen_t len = Fill(&addr, name);
    if (connect(s, reinterpret_cast<struct sockaddr*>(&addr), len) == 0) {
      sock_ = s;
      return;
    }
    close(s);
    if (std::chrono::steady_clock::now() > deadline)
      IBCOMM_FAIL(TRANSPORT_ERROR, "connect(@%s) failed: %s\n", name.c_str(), strerror(errno));
    std::this_thread::sleep_for(std::chrono::milliseconds(2));
  }
}

void FdChannel::Send(const void* payload, size_t len, int fd) {
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  struct iovec iov;
  iov.iov_base = const_cast<void*>(payload);
  iov.iov_len = len;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(struct cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  if (fd >= 0) {
    memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  ssize_t n;
  do {
    n = sendmsg(sock_, &msg, MSG_NOSIGNAL);
  } while (n < 0 && errno == EINTR);
  if (n != static_cast<ssize_t>(len)) IBCOMM_FAIL(TRANSPORT_ERROR, "sendmsg on the descriptor channel failed: %s\n", strerror(errno));
}

int FdChannel::Recv(void* payload, size_t len, int timeout_ms) {
  struct pollfd p = {sock_, POLLIN, 0};
  int rc = poll(&p, 1, timeout_ms);
  if (rc <= 0) IBCOMM_FAIL(TRANSPORT_ERROR, "Nothing arrived on the descriptor channel within %d ms.\n", timeout_ms);
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  struct iovec iov;
  iov.iov_base = payload;
  iov.iov_len = len;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  alignas(struct cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  ssize_t n;
  do {
    n = recvmsg(sock_, &msg, MSG_CMSG_CLOEXEC | MSG_WAITALL);
  } while (n < 0 && errno == EINTR);
  if (n != static_cast<ssize_t>(len))
    IBCOMM_FAIL(TRANSPORT_ERROR, "recvmsg on the descriptor channel returned %zd of %zu bytes.\n", n, len);
  int fd = -1;
  for (struct cmsghdr* c = CMSG_FIRSTHDR(&msg); c != nullptr; c = CMSG_NXTHDR(&msg, c)) {
    if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
      memcpy(&fd, CMSG_DATA(c), sizeof(int));
      break;
    }
  }
  return fd;
}

}  // namespace ibcomm
