// File-descriptor passing between the processes (or threads) of one host.
//
// Device allocations made with the virtual-memory API are shared by POSIX file
// descriptor, and a descriptor can only cross a process boundary as SCM_RIGHTS
// ancillary data on a unix-domain socket.  Each rank pair opens one stream
// socket (abstract namespace, named after the listening side's endpoint); the
// lower rank listens, the higher rank connects.
#pragma once

#include <cstddef>
#include <string>

namespace ibcomm {

class FdChannel {
 public:
  FdChannel() = default;
  ~FdChannel();
  FdChannel(const FdChannel&) = delete;
  FdChannel& operator=(const FdChannel&) = delete;

  // Server side, step 1: bind + listen on the abstract name.
  void Listen(const std::string& name);
  // Server side, step 2: accept the single client (bounded wait).
  void Accept(int timeout_ms);
  // Client side: connect to a listening name (retries until the limit).
  void Connect(const std::string& name, int timeout_ms);

  // One message = `len` payload bytes plus an optional descriptor (-1: none).
  void Send(const void* payload, size_t len, int fd);
  // Returns the received descriptor or -1.
  int Recv(void* payload, size_t len, int timeout_ms);

  bool connected() const { return sock_ >= 0; }

 private:
  int listen_fd_ = -1;
  int sock_ = -1;
};

std::string FdChannelName(unsigned pid, unsigned nonce);

}  // namespace ibcomm
