"""B200-native AllReduce library with the capabilities of PFN's allreduce
prototype ("ibcomm"): a communicator with two-sided messaging and ring /
Rabenseifner allreduce over host buffers, and hand-written sm_100a kernels for
device buffers (chunk-pipelined ring, recursive halving/doubling for any world
size, in-switch NVLS reduction, one-shot for small messages) with the sum, the
scale and the 16-bit wire cast fused.

    import allreduce_proto_b200 as ar
    comm = ar.Communicator.from_torch_distributed()
    comm.allreduce(grads, scale=1.0 / comm.world_size)
"""
from ._native import (CUDA_ERROR, IBVERBS_ERROR, INVALID_ARGUMENT, NOT_SUPPORTED, TRANSPORT_ERROR, IbcommError)
from .parallel import Communicator, EmuWorld, GradientBuckets, plan_buckets
from . import models, ops, parallel, utils

__all__ = ["Communicator", "EmuWorld", "GradientBuckets", "plan_buckets", "IbcommError", "INVALID_ARGUMENT",
           "TRANSPORT_ERROR", "IBVERBS_ERROR", "CUDA_ERROR", "NOT_SUPPORTED", "models", "ops", "parallel", "utils"]
__version__ = "0.1.0"
