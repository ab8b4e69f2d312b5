"""The chunk partitioner and the op programs, exposed for inspection and tests."""
from __future__ import annotations

import ctypes as C

from .. import _native


def split_buffer(len_elements: int, elem_bytes: int, world_size: int, chunk_bytes: int = 0):
    """Chunk ranges ``[(begin, end), ...]`` in elements (reference ibverbs_communicator.cpp:637-683).

    ``chunk_bytes <= 0`` means IBCOMM_CHUNKSIZE unset (4 * world_size chunks).
    Raises :class:`IbcommError` with code 1 or 4 for the reference's error cases.
    """
    cap = max(4 * world_size, 16)
    while True:
        pairs = (C.c_uint64 * (2 * cap))()
        count = C.c_size_t(0)
        _native.check(_native.lib().ibcomm_split_buffer(len_elements, elem_bytes, world_size, chunk_bytes, pairs, cap,
                                                         C.byref(count)))
        if count.value <= cap:
            return [(pairs[2 * i], pairs[2 * i + 1]) for i in range(count.value)]
        cap = count.value


def rank_to_chunk(num_chunks: int, world_size: int, rank: int):
    """Chunk ids owned by ``rank`` (contiguous blocks, reference ibverbs_communicator.cpp:685-707)."""
    cap = num_chunks + 1
    ids = (C.c_int * cap)()
    count = C.c_size_t(0)
    _native.check(_native.lib().ibcomm_rank_to_chunk(num_chunks, world_size, rank, ids, cap, C.byref(count)))
    return [ids[i] for i in range(count.value)]


def describe_program(algo: str, rank: int, world_size: int, len_elements: int, elem_bytes: int = 4,
                     chunk_bytes: int = 0, stage_bytes: int = 64 << 20) -> list[str]:
    """One line per op of the device program of ``rank``."""
    buf = C.create_string_buffer(1 << 20)
    _native.check(_native.lib().ibcomm_describe_program(_native.ALGO_CODES[algo], rank, world_size, len_elements,
                                                         elem_bytes, chunk_bytes, stage_bytes, buf, len(buf)))
    return [ln for ln in buf.value.decode().splitlines() if ln]
