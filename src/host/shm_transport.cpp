#include "ibcomm/shm_transport.h"

#include <errno.h>
#include <fcntl.h>
#include <signal.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "ibcomm/error.h"

namespace ibcomm {

std::string ShmName(uint32_t pid, uint32_t nonce) {
  char buf[64];
  snprintf(buf, sizeof(buf), "/ibcomm.%u.%08x", pid, nonce);
  return buf;
}

size_t ShmRingBytesFromEnv() {
  const char* s = getenv("IBCOMM_SHM_RING_BYTES");
  long long v = s ? atoll(s) : 0;
  if (v < 4096) v = 4ll << 20;
  return (static_cast<size_t>(v) + 4095) & ~size_t(4095);
}

static bool ProcessAlive(int pid) {
  if (pid <= 0) return true;
  return kill(pid, 0) == 0 || errno != ESRCH;
}

// ---------------------------------------------------------------- inbox
void ShmInbox::Create(const std::string& name, size_t capacity) {
  capacity = (capacity + 4095) & ~size_t(4095);
  size_t bytes = offsetof(ShmRingHeader, data) + capacity;
  int fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) IBCOMM_FAIL(TRANSPORT_ERROR, "shm_open(%s) failed: %s\n", name.c_str(), strerror(errno));
  if (ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
    int e = errno;
    close(fd);
    shm_unlink(name.c_str());
    IBCOMM_FAIL(TRANSPORT_ERROR, "ftruncate(%s, %zu) failed: %s\n", name.c_str(), bytes, strerror(e));
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) {
    shm_unlink(name.c_str());
    IBCOMM_FAIL(TRANSPORT_ERROR, "mmap(%s) failed: %s\n", name.c_str(), strerror(errno));
  }
  hdr_ = static_cast<ShmRingHeader*>(p);
  map_bytes_ = bytes;
  name_ = name;
  linked_ = true;
  hdr_->version = 1;
  hdr_->capacity = capacity;
  hdr_->owner_pid = getpid();
  hdr_->producer_pid.store(0, std::memory_order_relaxed);
  hdr_->consumer_gone.store(0, std::memory_order_relaxed);
  hdr_->producer_gone.store(0, std::memory_order_relaxed);
  hdr_->head.store(0, std::memory_order_relaxed);
  hdr_->tail.store(0, std::memory_order_relaxed);
  std::atomic_thread_fence(std::memory_order_release);
  hdr_->magic = kShmMagic;
}

ShmInbox::~ShmInbox() {
  if (hdr_ != nullptr) {
    hdr_->consumer_gone.store(1, std::memory_order_release);
    munmap(hdr_, map_bytes_);
  }
  UnlinkName();
}

void ShmInbox::UnlinkName() {
  if (linked_) {
    shm_unlink(name_.c_str());
    linked_ = false;
  }
}

size_t ShmInbox::Available() const {
  uint64_t h = hdr_->head.load(std::memory_order_acquire);
  uint64_t t = hdr_->tail.load(std::memory_order_relaxed);
  return static_cast<size_t>(h - t);
}

const unsigned char* ShmInbox::Peek(size_t* contiguous) const {
  uint64_t h = hdr_->head.load(std::memory_order_acquire);
  uint64_t t = hdr_->tail.load(std::memory_order_relaxed);
  size_t off = static_cast<size_t>(t % hdr_->capacity);
  size_t avail = static_cast<size_t>(h - t);
  *contiguous = std::min(avail, static_cast<size_t>(hdr_->capacity) - off);
  return hdr_->data + off;
}

void ShmInbox::Release(size_t bytes) {
  hdr_->tail.store(hdr_->tail.load(std::memory_order_relaxed) + bytes, std::memory_order_release);
}

bool ShmInbox::PeerDead() const {
  if (hdr_->producer_gone.load(std::memory_order_acquire)) return true;
  return !ProcessAlive(hdr_->producer_pid.load(std::memory_order_relaxed));
}

// ---------------------------------------------------------------- outbox
bool ShmOutbox::Open(const std::string& name) {
  int fd = shm_open(name.c_str(), O_RDWR, 0600);
  if (fd < 0) return false;
  struct stat st;
  if (fstat(fd, &st) != 0 || static_cast<size_t>(st.st_size) < sizeof(ShmRingHeader)) {
    close(fd);
    return false;
  }
  void* p = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) return false;
  ShmRingHeader* h = static_cast<ShmRingHeader*>(p);
  if (h->magic != kShmMagic) {
    munmap(p, static_cast<size_t>(st.st_size));
    return false;
  }
  hdr_ = h;
  map_bytes_ = static_cast<size_t>(st.st_size);
  local_head_ = hdr_->head.load(std::memory_order_relaxed);
  hdr_->producer_pid.store(getpid(), std::memory_order_release);
  return true;
}

ShmOutbox::~ShmOutbox() {
  if (hdr_ != nullptr) {
    hdr_->producer_gone.store(1, std::memory_order_release);
    munmap(hdr_, map_bytes_);
  }
}

size_t ShmOutbox::Space() const {
  uint64_t t = hdr_->tail.load(std::memory_order_acquire);
  return static_cast<size_t>(hdr_->capacity - (local_head_ - t));
}

size_t ShmOutbox::Write(const void* src, size_t n) {
  n = std::min(n, Space());
  const unsigned char* s = static_cast<const unsigned char*>(src);
  size_t left = n;
  while (left > 0) {
    size_t off = static_cast<size_t>(local_head_ % hdr_->capacity);
    size_t run = std::min(left, static_cast<size_t>(hdr_->capacity) - off);
    memcpy(hdr_->data + off, s, run);
    s += run;
    left -= run;
    local_head_ += run;
  }
  return n;
}

bool ShmOutbox::Pad(size_t n) {
  static const unsigned char zeros[kFrameAlign] = {0};
  if (n == 0) return true;
  if (Space() < n) return false;
  Write(zeros, n);
  return true;
}

void ShmOutbox::Publish() { hdr_->head.store(local_head_, std::memory_order_release); }

bool ShmOutbox::PeerDead() const {
  if (hdr_->consumer_gone.load(std::memory_order_acquire)) return true;
  return !ProcessAlive(hdr_->owner_pid);
}

}  // namespace ibcomm
