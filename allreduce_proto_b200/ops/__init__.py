"""Operations: allreduce and the fused copy/scale/cast kernel."""
from .allreduce import allreduce, copy_scale, default_communicator, init

__all__ = ["allreduce", "copy_scale", "init", "default_communicator"]
