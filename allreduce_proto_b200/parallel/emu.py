"""Several ranks on one GPU (``ibcomm::EmuWorld``): every collective is one
cooperative kernel launch that covers all ranks, so the real kernels, programs
and flag protocol can be exercised on a single-GPU machine."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .. import _native
from .._native import ALGO_CODES, check
from .communicator import _ptr, dtype_code


class EmuWorld:
    def __init__(self, num_ranks: int, pool_bytes: int = 0, work_bytes: int = 0):
        self._h = C.c_void_p()
        check(_native.lib().ibcomm_emu_create(num_ranks, pool_bytes, work_bytes, C.byref(self._h)))
        self.num_ranks = num_ranks

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            _native.lib().ibcomm_emu_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def allreduce(self, sendbufs: Sequence[torch.Tensor], recvbufs: Optional[Sequence[torch.Tensor]] = None, *,
                  algo: str = "ring", scale: float = 1.0, wire=None, channels: int = 0,
                  stream: Optional[torch.cuda.Stream] = None, sync: bool = True):
        """``recvbufs[r]`` = scale * sum over r of ``sendbufs[r]`` for every emulated rank."""
        if recvbufs is None:
            recvbufs = sendbufs
        n = sendbufs[0].numel()
        d = dtype_code(sendbufs[0].dtype)
        w = dtype_code(wire) if wire is not None else d
        ins = (C.c_void_p * self.num_ranks)(*[_ptr(t) for t in sendbufs])
        outs = (C.c_void_p * self.num_ranks)(*[_ptr(t) for t in recvbufs])
        s = stream if stream is not None else torch.cuda.current_stream()
        check(_native.lib().ibcomm_emu_allreduce(self._h, ALGO_CODES[algo], d, ins, outs, n, float(scale), w, channels,
                                                 C.c_void_p(s.cuda_stream), 0 if sync else 1))
        return recvbufs

    def reduce_scatter(self, sendbufs: Sequence[torch.Tensor], recvbufs: Sequence[torch.Tensor], *, scale: float = 1.0,
                       channels: int = 0):
        """``recvbufs[r]`` = scale * sum over ranks q of block r of ``sendbufs[q]`` (direct algorithm)."""
        return self._rsag(0, sendbufs, recvbufs, recvbufs[0].numel(), scale, channels)

    def all_gather(self, sendbufs: Sequence[torch.Tensor], recvbufs: Sequence[torch.Tensor], *, channels: int = 0):
        """Block q of every ``recvbufs[r]`` = ``sendbufs[q]`` (direct algorithm)."""
        return self._rsag(1, sendbufs, recvbufs, sendbufs[0].numel(), 1.0, channels)

    def _rsag(self, all_gather, sendbufs, recvbufs, block, scale, channels):
        d = dtype_code(sendbufs[0].dtype)
        ins = (C.c_void_p * self.num_ranks)(*[_ptr(t) for t in sendbufs])
        outs = (C.c_void_p * self.num_ranks)(*[_ptr(t) for t in recvbufs])
        s = torch.cuda.current_stream()
        check(_native.lib().ibcomm_emu_rsag(self._h, all_gather, d, ins, outs, block, float(scale), channels,
                                            C.c_void_p(s.cuda_stream), 0))
        return recvbufs

    def set_timeout_ms(self, ms: int) -> None:
        check(_native.lib().ibcomm_emu_set_timeout_ms(self._h, ms))

    def set_silent_rank(self, rank: int) -> None:
        """Test hook: ``rank`` skips the following collectives (-1: nobody does)."""
        check(_native.lib().ibcomm_emu_set_silent_rank(self._h, rank))

    def set_bad_program_rank(self, rank: int) -> None:
        """Test hook: ``rank`` fails the executor's per-op bounds check (-1: nobody does)."""
        check(_native.lib().ibcomm_emu_set_bad_program_rank(self._h, rank))

    def set_direct_staging(self, mode) -> None:
        """Direct algorithm: 0/False in place, 1/True staged through the pool windows one phase after the other,
        2 staged through the pipelined kernel (needs 16-byte aligned buffers of whole 16-byte vectors)."""
        check(_native.lib().ibcomm_emu_set_direct_staging(self._h, int(mode)))

    @property
    def last_channels(self) -> int:
        return _native.lib().ibcomm_emu_last_channels(self._h)

    def last_status(self) -> dict:
        rep = _native.StatusReport()
        check(_native.lib().ibcomm_emu_last_status(self._h, C.byref(rep)))
        return {f: getattr(rep, f) for f, _ in rep._fields_}
