// Host transport: one single-producer/single-consumer byte ring in POSIX
// shared memory per ordered rank pair.  It replaces the reference's RC queue
// pair (ibverbs_communicator.cpp:286-357): the receiver creates the ring
// ("inbox") and publishes its name through ProcessInfo; the sender attaches to
// it ("outbox").  Messages are framed (16-byte header with the payload length)
// and delivered strictly FIFO, so two-sided matching needs no tags.
#pragma once

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <string>

namespace ibcomm {

struct alignas(64) ShmRingHeader {
  uint32_t magic;
  uint32_t version;
  uint64_t capacity;              // bytes in data[], multiple of 16
  int32_t owner_pid;              // consumer (creator)
  std::atomic<int32_t> producer_pid;   // 0 until a sender attached
  std::atomic<uint32_t> consumer_gone; // set by the creator's destructor
  std::atomic<uint32_t> producer_gone; // set by the sender's destructor
  alignas(64) std::atomic<uint64_t> head;  // total bytes published by the producer
  alignas(64) std::atomic<uint64_t> tail;  // total bytes released by the consumer
  alignas(64) unsigned char data[1];
};

constexpr uint32_t kShmMagic = 0x1BC0223Du;
constexpr size_t kFrameAlign = 16;

std::string ShmName(uint32_t pid, uint32_t nonce);
size_t ShmRingBytesFromEnv();  // IBCOMM_SHM_RING_BYTES, default 4 MiB

// Receiver side.  Owns the mapping and the name.
class ShmInbox {
 public:
  ShmInbox() = default;
  ~ShmInbox();
  ShmInbox(const ShmInbox&) = delete;
  ShmInbox& operator=(const ShmInbox&) = delete;

  void Create(const std::string& name, size_t capacity);
  bool valid() const { return hdr_ != nullptr; }
  // Bytes published and not yet released.
  size_t Available() const;
  // Pointer to the first readable byte and the contiguous run length there.
  const unsigned char* Peek(size_t* contiguous) const;
  void Release(size_t bytes);
  // True when the sender has detached or its process no longer exists.
  bool PeerDead() const;
  const std::string& name() const { return name_; }
  void UnlinkName();

 private:
  ShmRingHeader* hdr_ = nullptr;
  size_t map_bytes_ = 0;
  std::string name_;
  bool linked_ = false;
};

// Sender side.
class ShmOutbox {
 public:
  ShmOutbox() = default;
  ~ShmOutbox();
  ShmOutbox(const ShmOutbox&) = delete;
  ShmOutbox& operator=(const ShmOutbox&) = delete;

  // Fails (returns false) when the name does not exist.
  bool Open(const std::string& name);
  bool valid() const { return hdr_ != nullptr; }
  size_t Space() const;
  // Writes up to n bytes without publishing; returns bytes written.
  size_t Write(const void* src, size_t n);
  // Writes n zero bytes (n <= 15) for frame padding; false if no space.
  bool Pad(size_t n);
  void Publish();
  bool PeerDead() const;

 private:
  ShmRingHeader* hdr_ = nullptr;
  size_t map_bytes_ = 0;
  uint64_t local_head_ = 0;  // written, possibly unpublished
};

}  // namespace ibcomm
