"""Operations: allreduce, its halves, and the fused copy/scale/cast kernel."""
from .allreduce import all_gather, allreduce, copy_scale, default_communicator, init, reduce_scatter

__all__ = ["allreduce", "reduce_scatter", "all_gather", "copy_scale", "init", "default_communicator"]
