"""Python face of ``ibcomm::Communicator`` for PyTorch programs.

One process per GPU.  The communicator keeps the reference's three-call
connection protocol (``create_queue_pair`` / exchange / ``register_queue_pair``,
reference ibcomm/ibverbs_communicator.h:84-87); :meth:`Communicator.from_torch_distributed`
runs it through the ``torch.distributed`` store so that a ``torchrun`` job needs
one line to get a communicator.  Tensors are passed by pointer; nothing is
copied on the way into the kernels.
"""
from __future__ import annotations

import ctypes as C
import os
import time
from typing import Optional, Sequence

import torch

from .. import _native
from .._native import ALGO_CODES, ALGO_NAMES, DTYPE_CODES, IbcommError, check

_TORCH_DTYPES = {
    torch.float32: "float32", torch.float64: "float64", torch.int32: "int32", torch.int64: "int64",
    torch.float16: "float16", torch.bfloat16: "bfloat16",
}


def dtype_code(dtype) -> int:
    if isinstance(dtype, str):
        return DTYPE_CODES[dtype]
    try:
        return DTYPE_CODES[_TORCH_DTYPES[dtype]]
    except KeyError:
        raise IbcommError(_native.NOT_SUPPORTED, f"unsupported dtype {dtype}") from None


def _ptr(t: torch.Tensor) -> int:
    if not t.is_contiguous():
        raise IbcommError(_native.INVALID_ARGUMENT, "tensors must be contiguous")
    return t.data_ptr()


class _CudaArray:
    """Minimal ``__cuda_array_interface__`` carrier for memory the library owns."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
        self._owner = owner


class Communicator:
    """AllReduce communicator of one rank.

    >>> comm = Communicator.from_torch_distributed()
    >>> comm.allreduce(grad, scale=1.0 / comm.world_size)   # in place, on the current stream
    """

    def __init__(self, world_size: int, rank: Optional[int] = None):
        self._h = C.c_void_p()
        check(_native.lib().ibcomm_create(world_size, C.byref(self._h)))
        self.world_size = world_size
        self.rank = -1
        self._symmetric = []
        self._registered = {}
        if rank is not None:
            self.register_myself(rank)

    # ------------------------------------------------------------ lifecycle
    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            lib = _native.lib()
            lib.ibcomm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self) -> "Communicator":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def __repr__(self) -> str:
        state = "open" if getattr(self, "_h", None) else "closed"
        return f"Communicator(world_size={self.world_size}, rank={getattr(self, 'rank', None)}, {state})"

    # --------------------------------------------------- connection protocol
    def create_queue_pair(self, dest_rank: int) -> tuple[int, int, int]:
        out = (C.c_uint32 * 3)()
        check(_native.lib().ibcomm_create_queue_pair(self._h, dest_rank, out))
        return (out[0], out[1], out[2])

    def register_queue_pair(self, dest_rank: int, info: Sequence[int]) -> None:
        arr = (C.c_uint32 * 3)(*info)
        check(_native.lib().ibcomm_register_queue_pair(self._h, dest_rank, arr))

    def register_process(self, dest_rank: int, info: Sequence[int]) -> tuple[int, int, int]:
        arr = (C.c_uint32 * 3)(*info)
        out = (C.c_uint32 * 3)()
        check(_native.lib().ibcomm_register_process(self._h, dest_rank, arr, out))
        return (out[0], out[1], out[2])

    def register_myself(self, rank: int) -> None:
        check(_native.lib().ibcomm_register_myself(self._h, rank))
        self.rank = rank

    def set_timeout_ms(self, ms: int) -> None:
        check(_native.lib().ibcomm_set_timeout_ms(self._h, ms))

    def set_max_channels(self, channels: int) -> None:
        """Caps the CTAs a collective may use (0 = IBCOMM_NUM_CUDA_STREAM)."""
        check(_native.lib().ibcomm_set_max_channels(self._h, channels))

    def connect_with(self, exchange) -> None:
        """Full-mesh connection.  ``exchange(rank, infos)`` receives this rank's
        ``{dest: info}`` and must return ``{src: info addressed to this rank}``."""
        mine = {d: self.create_queue_pair(d) for d in range(self.world_size) if d != self.rank}
        theirs = exchange(self.rank, mine)
        for src, info in theirs.items():
            self.register_queue_pair(src, info)
        # Nobody may leave (and take its endpoints away) before everybody attached.
        self.barrier()

    @classmethod
    def from_torch_distributed(cls, group=None, tag: str = "c0", ranks=None) -> "Communicator":
        """Builds a connected communicator from an initialised ``torch.distributed`` job.

        The descriptors travel through the job's key-value store (host only; no
        collective of the backend is used).

        ``ranks``: build the communicator over this subset of the job's ranks only (every member
        calls with the same list; the other ranks do not call); a rank's number in the new
        communicator is its position in the list."""
        import torch.distributed as dist
        if not dist.is_initialized():
            raise IbcommError(_native.INVALID_ARGUMENT, "torch.distributed is not initialised")
        rank, ws = dist.get_rank(group), dist.get_world_size(group)
        if ranks is not None:
            ranks = [int(r) for r in ranks]
            if rank not in ranks or len(set(ranks)) != len(ranks) or any(r < 0 or r >= ws for r in ranks):
                raise IbcommError(_native.INVALID_ARGUMENT, f"rank {rank} builds a communicator over {ranks}")
            tag = f"{tag}.sub" + "_".join(str(r) for r in ranks)
            rank, ws = ranks.index(rank), len(ranks)
        comm = cls(ws, rank)
        if ws == 1:
            return comm
        store = dist.distributed_c10d._get_default_store()

        def exchange(me, mine):
            for d, info in mine.items():
                store.set(f"ibcomm/{tag}/{me}/{d}", ",".join(str(v) for v in info))
            out = {}
            for s in range(ws):
                if s != me:
                    out[s] = tuple(int(v) for v in store.get(f"ibcomm/{tag}/{s}/{me}").decode().split(","))
            return out

        comm.connect_with(exchange)
        return comm

    @classmethod
    def from_env(cls, tag: str = "c0", timeout_s: float = 60.0, ranks=None) -> "Communicator":
        """Builds a connected communicator from the launcher's environment
        (``IBCOMM_RANK``/``RANK``, ``IBCOMM_WORLD_SIZE``/``WORLD_SIZE``, ``IBCOMM_BOOTSTRAP_DIR``),
        exchanging descriptors through files like the C++ ``ConnectAll``.

        ``ranks``: build the communicator over this subset of the job's ranks only (every member
        calls with the same list and a ``tag`` not used before); a rank's number in the new
        communicator is its position in the list.  This is how the survivors of a failed rank form
        a smaller world and carry on (the collectives of the old communicator have returned
        TRANSPORT_ERROR by then)."""
        rank = int(os.environ.get("IBCOMM_RANK", os.environ.get("RANK", "0")))
        ws = int(os.environ.get("IBCOMM_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
        if ranks is not None:
            ranks = [int(r) for r in ranks]
            if rank not in ranks or len(set(ranks)) != len(ranks) or any(r < 0 or r >= ws for r in ranks):
                raise IbcommError(_native.INVALID_ARGUMENT, f"rank {rank} builds a communicator over {ranks}")
            tag = f"{tag}.sub" + "_".join(str(r) for r in ranks)
            rank, ws = ranks.index(rank), len(ranks)
        comm = cls(ws, rank)
        if ws == 1:
            return comm
        d = os.environ.get("IBCOMM_BOOTSTRAP_DIR")
        if not d:
            raise IbcommError(_native.INVALID_ARGUMENT, "IBCOMM_BOOTSTRAP_DIR is not set")

        def exchange(me, mine):
            for dst, info in mine.items():
                path = os.path.join(d, f"{tag}.qp.{me}.{dst}")
                with open(path + ".tmp", "w") as f:
                    f.write("%d %d %d\n" % info)
                os.replace(path + ".tmp", path)
            out = {}
            deadline = time.time() + timeout_s
            for s in range(ws):
                if s == me:
                    continue
                path = os.path.join(d, f"{tag}.qp.{s}.{me}")
                while not os.path.exists(path):
                    if time.time() > deadline:
                        raise IbcommError(_native.TRANSPORT_ERROR, f"rank {s} never published its endpoint")
                    time.sleep(0.001)
                with open(path) as f:
                    out[s] = tuple(int(v) for v in f.read().split())
            return out

        comm.connect_with(exchange)
        return comm

    # ------------------------------------------------------------ messaging
    @staticmethod
    def _buf(t):
        if isinstance(t, torch.Tensor):
            return _ptr(t), t.numel() * t.element_size()
        import numpy as np
        a = np.ascontiguousarray(t) if not (hasattr(t, "flags") and t.flags["C_CONTIGUOUS"]) else t
        return a.ctypes.data, a.nbytes

    def send(self, dest_rank: int, tensor, blocking: bool = True) -> None:
        p, n = self._buf(tensor)
        check(_native.lib().ibcomm_send(self._h, dest_rank, p, n, int(blocking)))

    def recv(self, src_rank: int, tensor, blocking: bool = True) -> None:
        p, n = self._buf(tensor)
        check(_native.lib().ibcomm_recv(self._h, src_rank, p, n, int(blocking)))

    def send_poll(self, dest_rank: int) -> bool:
        done = C.c_int(0)
        check(_native.lib().ibcomm_send_poll(self._h, dest_rank, C.byref(done)))
        return bool(done.value)

    def recv_poll(self, src_rank: int) -> bool:
        done = C.c_int(0)
        check(_native.lib().ibcomm_recv_poll(self._h, src_rank, C.byref(done)))
        return bool(done.value)

    def send_wait(self, dest_rank: int) -> None:
        check(_native.lib().ibcomm_send_wait(self._h, dest_rank))

    def recv_wait(self, src_rank: int) -> None:
        check(_native.lib().ibcomm_recv_wait(self._h, src_rank))

    def bcast(self, tensor, root: int) -> None:
        p, n = self._buf(tensor)
        check(_native.lib().ibcomm_bcast(self._h, p, n, root))

    def barrier(self) -> None:
        check(_native.lib().ibcomm_barrier(self._h))

    # ------------------------------------------------------------ allreduce
    def allreduce(self, sendbuf: torch.Tensor, recvbuf: Optional[torch.Tensor] = None, *, algo: str = "auto",
                  scale: float = 1.0, wire=None, stream: Optional[torch.cuda.Stream] = None,
                  sync: bool = False) -> torch.Tensor:
        """Sum of ``sendbuf`` over all ranks (times ``scale``) into ``recvbuf`` (default: in place).

        CUDA tensors run on ``stream`` (default: the current stream) and the call
        only enqueues unless ``sync``; CPU tensors use the host transport and
        return when done.  ``wire`` = ``torch.bfloat16`` / ``torch.float16`` sends
        fp32 data in 16 bits (sums are accumulated in fp32)."""
        if recvbuf is None:
            recvbuf = sendbuf
        if sendbuf.dtype != recvbuf.dtype or sendbuf.numel() != recvbuf.numel():
            raise IbcommError(_native.INVALID_ARGUMENT, "sendbuf and recvbuf must match in dtype and size")
        d = dtype_code(sendbuf.dtype)
        lib = _native.lib()
        if not sendbuf.is_cuda:
            if recvbuf.is_cuda:
                raise IbcommError(_native.INVALID_ARGUMENT, "sendbuf and recvbuf must live on the same kind of device")
            a = ALGO_CODES["ring" if algo == "auto" else algo]
            check(lib.ibcomm_allreduce_host(self._h, a, d, _ptr(sendbuf), _ptr(recvbuf), sendbuf.numel()))
            if scale != 1.0:
                recvbuf.mul_(scale)
            return recvbuf
        w = dtype_code(wire) if wire is not None else d
        s = stream if stream is not None else torch.cuda.current_stream(sendbuf.device)
        check(lib.ibcomm_allreduce_cuda(self._h, ALGO_CODES[algo], d, _ptr(sendbuf), _ptr(recvbuf), sendbuf.numel(),
                                        float(scale), w, C.c_void_p(s.cuda_stream), 2 | (0 if sync else 1)))
        return recvbuf

    def reduce_scatter(self, sendbuf: torch.Tensor, recvbuf: torch.Tensor, *, algo: str = "auto", scale: float = 1.0,
                       stream: Optional[torch.cuda.Stream] = None, sync: bool = False) -> torch.Tensor:
        """``recvbuf`` = ``scale`` * sum over ranks of block ``rank`` of ``sendbuf``.

        ``sendbuf`` holds ``world_size`` blocks of ``recvbuf.numel()`` elements.  CUDA
        tensors: ``algo`` auto, nvls or direct; CPU tensors: a ring over the host transport.  ``recvbuf`` may be block ``rank`` of
        ``sendbuf`` (in place)."""
        if sendbuf.dtype != recvbuf.dtype or sendbuf.numel() != recvbuf.numel() * self.world_size:
            raise IbcommError(_native.INVALID_ARGUMENT, "sendbuf must hold world_size blocks of recvbuf's size and dtype")
        if sendbuf.is_cuda != recvbuf.is_cuda:
            raise IbcommError(_native.INVALID_ARGUMENT, "sendbuf and recvbuf must live on the same kind of device")
        if not sendbuf.is_cuda:
            check(_native.lib().ibcomm_reduce_scatter_host(self._h, dtype_code(sendbuf.dtype), _ptr(sendbuf), _ptr(recvbuf),
                                                           recvbuf.numel()))
            if scale != 1.0:
                recvbuf.mul_(scale)
            return recvbuf
        s = stream if stream is not None else torch.cuda.current_stream(sendbuf.device)
        check(_native.lib().ibcomm_reduce_scatter_cuda(self._h, ALGO_CODES[algo], dtype_code(sendbuf.dtype), _ptr(sendbuf),
                                                       _ptr(recvbuf), recvbuf.numel(), float(scale),
                                                       C.c_void_p(s.cuda_stream), 2 | (0 if sync else 1)))
        return recvbuf

    def all_gather(self, sendbuf: torch.Tensor, recvbuf: torch.Tensor, *, algo: str = "auto",
                   stream: Optional[torch.cuda.Stream] = None, sync: bool = False) -> torch.Tensor:
        """Block ``r`` of ``recvbuf`` = rank ``r``'s ``sendbuf`` (CUDA tensors: ``algo`` auto, nvls or direct;
        CPU tensors: a ring over the host transport).

        ``sendbuf`` may be block ``rank`` of ``recvbuf`` (in place)."""
        if sendbuf.dtype != recvbuf.dtype or recvbuf.numel() != sendbuf.numel() * self.world_size:
            raise IbcommError(_native.INVALID_ARGUMENT, "recvbuf must hold world_size blocks of sendbuf's size and dtype")
        if sendbuf.is_cuda != recvbuf.is_cuda:
            raise IbcommError(_native.INVALID_ARGUMENT, "sendbuf and recvbuf must live on the same kind of device")
        if not sendbuf.is_cuda:
            check(_native.lib().ibcomm_all_gather_host(self._h, dtype_code(sendbuf.dtype), _ptr(sendbuf), _ptr(recvbuf),
                                                       sendbuf.numel()))
            return recvbuf
        s = stream if stream is not None else torch.cuda.current_stream(sendbuf.device)
        check(_native.lib().ibcomm_all_gather_cuda(self._h, ALGO_CODES[algo], dtype_code(sendbuf.dtype), _ptr(sendbuf),
                                                   _ptr(recvbuf), sendbuf.numel(), C.c_void_p(s.cuda_stream),
                                                   2 | (0 if sync else 1)))
        return recvbuf

    def check(self) -> None:
        """Raises when an earlier asynchronous collective failed (call after synchronising)."""
        check(_native.lib().ibcomm_check(self._h))

    # ----------------------------------------------------- symmetric memory
    def symmetric_empty(self, numel: int, dtype=torch.float32) -> torch.Tensor:
        """A tensor in peer-mapped (and, with NVSwitch multicast, switch-reducible) memory.

        Collective: every rank must call with the same size in the same order.
        Allreduces whose buffers live in such tensors skip all staging copies."""
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        out = C.c_void_p()
        check(_native.lib().ibcomm_symmetric_alloc(self._h, max(nbytes, 16), C.byref(out)))
        raw = torch.as_tensor(_CudaArray(out.value, max(nbytes, 16), self), device=torch.device("cuda", torch.cuda.current_device()))
        self._symmetric.append(out.value)
        return raw[:nbytes].view(dtype)

    def register(self, tensor: torch.Tensor) -> int:
        """Maps an ordinary CUDA tensor of every rank (same byte size) into the peers.

        Collective.  Allreduces on the tensor (or on the same slice of it on every
        rank) then run without staging copies, like tensors from `symmetric_empty`
        but with peer loads/stores instead of the switch reduction.  Returns a
        registration id, or -1 (on every rank) when the allocator's memory cannot
        be shared through CUDA IPC (e.g. expandable segments); the tensor keeps
        working through the staging pool then.  The communicator holds a
        reference to the tensor until `deregister`."""
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError("register needs a contiguous CUDA tensor")
        rid = C.c_int(-1)
        check(_native.lib().ibcomm_register_buffer(self._h, C.c_void_p(tensor.data_ptr()),
                                                   tensor.numel() * tensor.element_size(), C.byref(rid)))
        if rid.value >= 0:
            self._registered[rid.value] = tensor
        return rid.value

    def deregister(self, rid: int) -> None:
        """Collective: drops a registration made by `register`."""
        if rid in self._registered:
            check(_native.lib().ibcomm_deregister_buffer(self._h, int(rid)))
            del self._registered[rid]

    def device_info(self, connect: bool = False) -> dict:
        info = _native.DeviceInfo()
        check(_native.lib().ibcomm_get_device_info(self._h, int(connect), C.byref(info)))
        return {"device": info.device, "nvls": bool(info.nvls), "share_mode": "vmm" if info.share_mode == 0 else "ipc",
                "last_algo": ALGO_NAMES.get(info.last_algo, "copy"), "last_channels": info.last_channels,
                "arena_bytes": info.arena_bytes, "pool_bytes": info.pool_bytes, "work_bytes": info.work_bytes,
                "calls": info.calls, "kernel_launches": info.kernel_launches,
                "switch_registrations": info.switch_registrations}

    # -------------------------------------------------------------- tracing
    def set_timer_base(self) -> None:
        check(_native.lib().ibcomm_set_timer_base(self._h))

    def dump_trace(self) -> None:
        check(_native.lib().ibcomm_dump_trace(self._h))

    def staged_timeline(self) -> dict:
        """Per-role device stamps of the last allreduce that ran the pipelined staged kernel with tracing on
        (``IBCOMM_TRACE=1``), CTA 0, in microseconds from the call's first stamp.  Per window: ``reduce`` =
        (waits satisfied, last store issued, window published), ``load`` = (input buffer free, input window
        published), ``store`` = (window reduced on every rank, output buffer released).  Empty without a trace."""
        cap = 8 * 128
        buf = (C.c_uint64 * cap)()
        words = C.c_size_t(0)
        check(_native.lib().ibcomm_staged_timeline(self._h, buf, cap, C.byref(words)))
        w = min(int(words.value), cap) // 8
        us = [v / 1e3 for v in buf[:8 * w]]
        pair = lambda role, k: (us[2 * (role * w + k)], us[2 * (role * w + k) + 1])  # noqa: E731
        return {"windows": w,
                "reduce": [(pair(0, k)[0], pair(3, k)[0], pair(0, k)[1]) for k in range(w)],
                "load": [pair(1, k) for k in range(w)],
                "store": [pair(2, k) for k in range(w)]}
