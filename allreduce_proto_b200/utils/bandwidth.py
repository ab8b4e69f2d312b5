"""Bandwidth arithmetic used by the benchmarks and the roofline reports."""
from __future__ import annotations


def algbw_gbs(bytes_per_rank: int, seconds: float) -> float:
    """Algorithm bandwidth: message bytes / time, in GB/s (1e9)."""
    return bytes_per_rank / seconds / 1e9


def busbw_gbs(bytes_per_rank: int, seconds: float, world_size: int) -> float:
    """Bus bandwidth of an allreduce: algbw * 2 * (n - 1) / n (algbw itself for n = 1)."""
    a = algbw_gbs(bytes_per_rank, seconds)
    return a if world_size <= 1 else a * 2.0 * (world_size - 1) / world_size


def ring_bytes_per_gpu(bytes_per_rank: int, world_size: int) -> float:
    """Bytes every GPU must send (and receive) in a ring or Rabenseifner allreduce."""
    return 2.0 * bytes_per_rank * (world_size - 1) / world_size


def nvls_bytes_per_gpu(bytes_per_rank: int, world_size: int) -> float:
    """Bytes per direction per GPU of the two-shot in-switch allreduce (about S * (1 + 1/n))."""
    return bytes_per_rank * (1.0 + 1.0 / world_size)
