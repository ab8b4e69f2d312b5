"""Host utilities: size strings, the buffer partitioner, bandwidth arithmetic."""
from .sizes import parse_number, get_exp_of_two, format_bytes
from .partition import split_buffer, rank_to_chunk, describe_program
from .bandwidth import algbw_gbs, busbw_gbs, ring_bytes_per_gpu, nvls_bytes_per_gpu
from .tuning import choose_algorithm, set_tunable, get_tunable
from .numa import device_numa_node, numa_node_of_device

__all__ = ["parse_number", "get_exp_of_two", "format_bytes", "split_buffer", "rank_to_chunk", "describe_program",
           "algbw_gbs", "busbw_gbs", "ring_bytes_per_gpu", "nvls_bytes_per_gpu", "choose_algorithm", "set_tunable", "get_tunable", "device_numa_node", "numa_node_of_device"]
