"""Functional entry points over a process-wide default communicator."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _native
from .._native import check
from ..parallel.communicator import Communicator, _ptr, dtype_code

_default: Optional[Communicator] = None


def init(comm: Optional[Communicator] = None) -> Communicator:
    """Sets (or builds from ``torch.distributed``) the default communicator."""
    global _default
    _default = comm if comm is not None else Communicator.from_torch_distributed()
    return _default


def default_communicator() -> Communicator:
    if _default is None:
        raise _native.IbcommError(_native.INVALID_ARGUMENT, "call allreduce_proto_b200.ops.init() first")
    return _default


def allreduce(tensor: torch.Tensor, out: Optional[torch.Tensor] = None, *, algo: str = "auto", scale: float = 1.0,
              wire=None, sync: bool = False, comm: Optional[Communicator] = None) -> torch.Tensor:
    """Sum over ranks (times ``scale``); in place unless ``out`` is given."""
    return (comm or default_communicator()).allreduce(tensor, out, algo=algo, scale=scale, wire=wire, sync=sync)


def reduce_scatter(tensor: torch.Tensor, out: torch.Tensor, *, algo: str = "auto", scale: float = 1.0,
                   sync: bool = False, comm: Optional[Communicator] = None) -> torch.Tensor:
    """``out`` = ``scale`` * sum over ranks of block ``rank`` of ``tensor`` (``world_size`` blocks)."""
    return (comm or default_communicator()).reduce_scatter(tensor, out, algo=algo, scale=scale, sync=sync)


def all_gather(tensor: torch.Tensor, out: torch.Tensor, *, algo: str = "auto", sync: bool = False,
               comm: Optional[Communicator] = None) -> torch.Tensor:
    """Block ``r`` of ``out`` = rank ``r``'s ``tensor``."""
    return (comm or default_communicator()).all_gather(tensor, out, algo=algo, sync=sync)


def copy_scale(src: torch.Tensor, dst: Optional[torch.Tensor] = None, scale: float = 1.0,
               out_dtype=None) -> torch.Tensor:
    """``dst = cast(src * scale)`` with the library's bulk-copy kernel (the
    world-size-1 path of the allreduce)."""
    if dst is None:
        dst = torch.empty_like(src, dtype=out_dtype or src.dtype)
    s = torch.cuda.current_stream(src.device)
    check(_native.lib().ibcomm_copy_scale(_ptr(src), _ptr(dst), src.numel(), dtype_code(src.dtype), dtype_code(dst.dtype),
                                          float(scale), C.c_void_p(s.cuda_stream)))
    return dst
