#include "ibcomm/partition.h"

#include <algorithm>

#include "ibcomm/env.h"
#include "ibcomm/error.h"
#include "ibcomm/util.h"

namespace ibcomm {

static void CheckLength(size_t len_elements, size_t world_size) {
  if (len_elements < world_size) {
    IBCOMM_FAIL(NOT_SUPPORTED,
                "Input vector is too short for the chunked Allreduce algorithms: %zu elements "
                "for %zu processes.\nUse at least as many elements as processes.\n",
                len_elements, world_size);
  }
}

static std::vector<Range> Cut(size_t len_elements, size_t sizeof_element, size_t world_size,
                              int64_t env_chunk_bytes) {
  size_t chunks;
  size_t per_chunk;
  if (env_chunk_bytes > 0) {
    if (static_cast<size_t>(env_chunk_bytes) % sizeof_element != 0) {
      IBCOMM_FAIL(INVALID_ARGUMENT,
                  "Selected `IBCOMM_CHUNKSIZE` (%lld) is not divisible by `sizeof(T)` (%zu).\n",
                  static_cast<long long>(env_chunk_bytes), sizeof_element);
    }
    per_chunk = static_cast<size_t>(env_chunk_bytes) / sizeof_element;
    chunks = util::ceilDiv(len_elements, per_chunk);
    if (chunks < 2 * world_size) {
      IBCOMM_FAIL(INVALID_ARGUMENT,
                  "Selected `IBCOMM_CHUNKSIZE` is too large.\n"
                  "Satisfy 2 * `world_size` <= `allreduce_bufsize` / `IBCOMM_CHUNKSIZE`.\n");
    }
  } else {
    chunks = 4 * world_size;
    per_chunk = util::ceilDiv(len_elements, chunks);
  }
  std::vector<Range> ranges;
  ranges.reserve(chunks);
  for (size_t i = 0; i < chunks; ++i) {
    size_t b = per_chunk * i;
    if (b >= len_elements) break;
    ranges.emplace_back(b, std::min(len_elements, b + per_chunk));
  }
  return ranges;
}

std::vector<Range> SplitBuffer(size_t len_elements, size_t sizeof_element, size_t world_size,
                               int64_t env_chunk_bytes) {
  CheckLength(len_elements, world_size);
  return Cut(len_elements, sizeof_element, world_size, env_chunk_bytes);
}

std::vector<Range> SplitBufferEnv(size_t len_elements, size_t sizeof_element, size_t world_size) {
  CheckLength(len_elements, world_size);
  return Cut(len_elements, sizeof_element, world_size, env::ReadChunkSize());
}

std::vector<std::vector<int>> GetRankToChunk(size_t num_chunks, size_t world_size) {
  std::vector<std::vector<int>> out(world_size);
  const size_t base = num_chunks / world_size;
  const size_t extra = num_chunks % world_size;
  int next = 0;
  for (size_t r = 0; r < world_size; ++r) {
    size_t n = base + (r < extra ? 1 : 0);
    out[r].reserve(n);
    for (size_t j = 0; j < n; ++j) out[r].push_back(next++);
  }
  return out;
}

std::vector<Range> SplitEven(size_t len_elements, size_t parts) {
  std::vector<Range> out;
  out.reserve(parts);
  for (size_t i = 0; i < parts; ++i) {
    size_t b = static_cast<size_t>((static_cast<unsigned __int128>(len_elements) * i) / parts);
    size_t e = static_cast<size_t>((static_cast<unsigned __int128>(len_elements) * (i + 1)) / parts);
    out.emplace_back(b, e);
  }
  return out;
}

}  // namespace ibcomm
