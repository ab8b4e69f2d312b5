"""Workload definitions (this is a collective library: the "models" are the
tensor shapes its benchmarks allreduce)."""
from .resnet50 import resnet50_num_params, resnet50_param_shapes, synthetic_grads

__all__ = ["resnet50_param_shapes", "resnet50_num_params", "synthetic_grads"]
