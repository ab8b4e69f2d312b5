// Staging pool with an exclusive lease: the public surface of the reference's
// pool layer (memory_pool.h:79-121 `MemoryPool::GetController`, :188-268
// `MemoryController::getMemory` / `returnMemory`) for callers that pipeline
// their own transfers through fixed-size slots.
//
// The collectives of this library do not go through it: their staging is the
// peer-mapped arena that the kernels address directly (src/cuda/arena.cpp,
// src/cuda/engine.cpp `ArenaLayout`), leased to one collective at a time by
// `Communicator::CollectiveLease`.  What this header keeps is the contract:
//
//   * a pool owns blocks of `IBCOMM_MEMORY_POOL_PRE_ALLOC` bytes and a set of
//     `IBCOMM_NUM_CUDA_STREAM` streams, both validated like the reference;
//   * `GetController(chunk_size)` hands out ONE controller at a time; a second
//     one while the first lives is NOT_SUPPORTED (exit code 4);
//   * the controller cuts every block into slots of `chunk_size` bytes and
//     hands them out first-in first-out, each paired with a stream;
//   * when the slots run out the pool allocates another block, and when the
//     streams run out it creates another stream: both with a warning here,
//     silently in the reference;
//   * returned slots and streams are reused in the order they came back.
//
// The block allocator and the stream factory are policies, so the same class
// serves host memory (tests, CPU transfers) and, under USE_CUDA, pinned or
// device memory with real CUDA streams.
#pragma once

#include <cstddef>
#include <cstdlib>
#include <deque>
#include <memory>
#include <utility>
#include <vector>

#include "ibcomm/env.h"
#include "ibcomm/error.h"

namespace ibcomm {

using StreamHandle = void*;

// One allocation of the pool.  Not copyable: slots point into it.
class MemoryBlock {
 public:
  MemoryBlock(void* ptr, size_t length) : ptr_(ptr), length_(length) {}
  MemoryBlock(const MemoryBlock&) = delete;
  MemoryBlock& operator=(const MemoryBlock&) = delete;
  void* ptr() const { return ptr_; }
  size_t length() const { return length_; }

 private:
  void* ptr_;
  size_t length_;
};

// One slot of `chunk_size` bytes inside a block, with the stream it is paired
// with while it is handed out (nullptr while it is vacant).
class Memory {
 public:
  Memory(MemoryBlock* block, size_t offset) : block_(block), offset_(offset), stream_(nullptr) {}
  void* ptr() const { return static_cast<char*>(block_->ptr()) + offset_; }
  size_t offset() const { return offset_; }
  const MemoryBlock* block() const { return block_; }
  StreamHandle stream() const { return stream_; }
  Memory* SetStream(StreamHandle s) {
    stream_ = s;
    return this;
  }
  Memory* UnsetStream() {
    stream_ = nullptr;
    return this;
  }

 private:
  MemoryBlock* block_;
  size_t offset_;
  StreamHandle stream_;
};

// Page-aligned host memory.
struct HostBlockAllocator {
  void* Allocate(size_t bytes) {
    void* p = nullptr;
    if (posix_memalign(&p, 4096, bytes < 4096 ? 4096 : bytes) != 0) return nullptr;
    return p;
  }
  void Free(void* p) { free(p); }
};

// Stream handles that are only tokens (1, 2, 3, ...): for host transfers.
struct TokenStreams {
  StreamHandle Create() { return reinterpret_cast<StreamHandle>(++next_); }
  void Destroy(StreamHandle) {}
  uintptr_t next_ = 0;
};

#ifdef USE_CUDA
// Page-locked host memory, mapped for the device.
struct PinnedBlockAllocator {
  void* Allocate(size_t bytes) {
    void* p = nullptr;
    CUDACHECK(cudaHostAlloc(&p, bytes, cudaHostAllocPortable));
    return p;
  }
  void Free(void* p) { cudaFreeHost(p); }
};
// Memory of the current device.
struct DeviceBlockAllocator {
  void* Allocate(size_t bytes) {
    void* p = nullptr;
    CUDACHECK(cudaMalloc(&p, bytes));
    return p;
  }
  void Free(void* p) { cudaFree(p); }
};
// Non-blocking CUDA streams (the reference's, memory_pool.h:94-96).
struct CudaStreams {
  StreamHandle Create() {
    cudaStream_t s;
    CUDACHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    return static_cast<StreamHandle>(s);
  }
  void Destroy(StreamHandle s) { cudaStreamDestroy(static_cast<cudaStream_t>(s)); }
};
#endif

template <class Allocator, class Streams>
class MemoryController;

template <class Allocator = HostBlockAllocator, class Streams = TokenStreams>
class MemoryPool {
  friend class MemoryController<Allocator, Streams>;

 public:
  // Block size and stream count from the environment (validated, exit code 1
  // outside 4..1 GiB and 1..1024), or given explicitly.
  MemoryPool() : MemoryPool(env::ReadPreAllocSize(), env::ReadNumCudaStream()) {}
  MemoryPool(size_t block_bytes, int num_streams) : block_bytes_(block_bytes) {
    if (block_bytes < 4 || block_bytes > (1ull << 30))
      IBCOMM_FAIL(INVALID_ARGUMENT, "Invalid block size for the memory pool: %zu\n", block_bytes);
    if (num_streams <= 0 || num_streams > 1024)
      IBCOMM_FAIL(INVALID_ARGUMENT, "Invalid number of streams for the memory pool: %d\n", num_streams);
    for (int i = 0; i < num_streams; ++i) streams_.push_back(stream_factory_.Create());
    Allocate();
  }
  MemoryPool(const MemoryPool&) = delete;
  MemoryPool& operator=(const MemoryPool&) = delete;
  ~MemoryPool() {
    for (StreamHandle s : streams_) stream_factory_.Destroy(s);
    for (auto& b : blocks_) allocator_.Free(b->ptr());
  }

  // The one controller of this pool; NOT_SUPPORTED while another one lives.
  MemoryController<Allocator, Streams> GetController(size_t chunk_size) {
    if (controller_in_use_) IBCOMM_FAIL(NOT_SUPPORTED, "Currently, MemoryController is in use.\n");
    if (chunk_size == 0 || chunk_size > block_bytes_)
      IBCOMM_FAIL(INVALID_ARGUMENT, "Chunk size %zu does not fit a pool block of %zu bytes.\n", chunk_size, block_bytes_);
    controller_in_use_ = true;
    return MemoryController<Allocator, Streams>(this, chunk_size);
  }

  size_t block_bytes() const { return block_bytes_; }
  size_t num_blocks() const { return blocks_.size(); }
  size_t num_streams() const { return streams_.size(); }
  bool controller_in_use() const { return controller_in_use_; }

 private:
  MemoryBlock* Allocate() {
    void* p = allocator_.Allocate(block_bytes_);
    if (p == nullptr) IBCOMM_FAIL(TRANSPORT_ERROR, "Cannot allocate a pool block of %zu bytes.\n", block_bytes_);
    if (!blocks_.empty())
      IBCOMM_WARN("memory pool: every slot is in use; allocated block %zu of %zu bytes.\n", blocks_.size() + 1, block_bytes_);
    blocks_.emplace_back(new MemoryBlock(p, block_bytes_));
    return blocks_.back().get();
  }
  StreamHandle AddStream() {
    IBCOMM_WARN("memory pool: every stream is in use; created stream %zu.\n", streams_.size() + 1);
    streams_.push_back(stream_factory_.Create());
    return streams_.back();
  }

  size_t block_bytes_;
  Allocator allocator_;
  Streams stream_factory_;
  std::vector<std::unique_ptr<MemoryBlock>> blocks_;
  std::vector<StreamHandle> streams_;
  bool controller_in_use_ = false;
};

template <class Allocator, class Streams>
class MemoryController {
 public:
  MemoryController(MemoryPool<Allocator, Streams>* pool, size_t chunk_size) : pool_(pool), chunk_size_(chunk_size) {
    if (pool == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "pool is nullptr.\n");
    for (StreamHandle s : pool_->streams_) vacant_streams_.push_back(s);
    for (auto& b : pool_->blocks_) Cut(b.get());
  }
  MemoryController(const MemoryController&) = delete;
  MemoryController& operator=(const MemoryController&) = delete;
  MemoryController(MemoryController&& o) noexcept { *this = std::move(o); }
  MemoryController& operator=(MemoryController&& o) noexcept {
    Release();
    pool_ = o.pool_;
    chunk_size_ = o.chunk_size_;
    slots_ = std::move(o.slots_);
    vacant_memories_ = std::move(o.vacant_memories_);
    vacant_streams_ = std::move(o.vacant_streams_);
    o.pool_ = nullptr;
    return *this;
  }
  ~MemoryController() { Release(); }

  // Oldest vacant slot paired with the oldest vacant stream; grows the pool
  // when either has run out.
  Memory* getMemory() {
    if (vacant_streams_.empty()) vacant_streams_.push_back(pool_->AddStream());
    StreamHandle s = vacant_streams_.front();
    vacant_streams_.pop_front();
    if (vacant_memories_.empty()) Cut(pool_->Allocate());
    Memory* m = vacant_memories_.front();
    vacant_memories_.pop_front();
    return m->SetStream(s);
  }
  void returnMemory(Memory* m) {
    if (m == nullptr || m->stream() == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "returnMemory: not a slot that is handed out.\n");
    vacant_streams_.push_back(m->stream());
    vacant_memories_.push_back(m->UnsetStream());
  }

  size_t chunk_size() const { return chunk_size_; }
  size_t vacant_slots() const { return vacant_memories_.size(); }
  size_t total_slots() const { return slots_.size(); }

 private:
  void Cut(MemoryBlock* b) {
    for (size_t off = 0; off + chunk_size_ <= b->length(); off += chunk_size_) {
      slots_.emplace_back(new Memory(b, off));
      vacant_memories_.push_back(slots_.back().get());
    }
  }
  void Release() {
    if (pool_ != nullptr) pool_->controller_in_use_ = false;
    pool_ = nullptr;
    slots_.clear();
    vacant_memories_.clear();
    vacant_streams_.clear();
  }

  MemoryPool<Allocator, Streams>* pool_ = nullptr;
  size_t chunk_size_ = 0;
  std::vector<std::unique_ptr<Memory>> slots_;
  std::deque<Memory*> vacant_memories_;
  std::deque<StreamHandle> vacant_streams_;
};

}  // namespace ibcomm
