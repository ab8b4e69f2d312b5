"""Communicators and data-parallel helpers."""
from .communicator import Communicator, dtype_code
from .emu import EmuWorld
from .buckets import GradientBuckets, plan_buckets

__all__ = ["Communicator", "EmuWorld", "GradientBuckets", "plan_buckets", "dtype_code"]
