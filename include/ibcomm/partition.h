// Buffer partitioner shared by every chunked allreduce schedule.
//
// A message of `len_elements` is cut into chunks (the pipeline unit); chunk
// ids are handed to ranks in contiguous blocks.  The cut, its validation and
// the exit codes reproduce the reference (ibverbs_communicator.cpp:637-707)
// with 64-bit element indices instead of `int`.
#pragma once

#include <cstddef>
#include <cstdint>
#include <utility>
#include <vector>

namespace ibcomm {

using Range = std::pair<size_t, size_t>;  // [first, second) in elements

// `env_chunk_bytes` <= 0 means "not set": 4 * world_size chunks of
// ceil(len / chunks) elements.  Otherwise the value must be a multiple of
// `sizeof_element` and give at least 2 * world_size chunks (INVALID_ARGUMENT).
// A message shorter than world_size elements is NOT_SUPPORTED.  Empty tail
// ranges are dropped, so a short message yields fewer than 4 * world_size.
std::vector<Range> SplitBuffer(size_t len_elements, size_t sizeof_element, size_t world_size,
                               int64_t env_chunk_bytes);

// Same, reading IBCOMM_CHUNKSIZE at the point of use like the reference does
// (after the length check).
std::vector<Range> SplitBufferEnv(size_t len_elements, size_t sizeof_element, size_t world_size);

// rank -> ascending chunk ids.  floor(chunks / ws) each, the first
// chunks % ws ranks get one more.
std::vector<std::vector<int>> GetRankToChunk(size_t num_chunks, size_t world_size);

// world_size equal element ranges (the last ones absorb nothing extra: range i
// is [i*len/ws, (i+1)*len/ws) computed in 128-bit so no overflow).  Used by
// the unchunked CPU Rabenseifner, which ignores IBCOMM_CHUNKSIZE
// (reference allreduce_cpu_impl.h:264-271).
std::vector<Range> SplitEven(size_t len_elements, size_t parts);

}  // namespace ibcomm
