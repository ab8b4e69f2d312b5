"""Gradient bucketing for data-parallel training (the use case the reference
names in its README.md:3-9 but leaves to the framework on top).

Gradients are packed into flat buckets of about ``bucket_bytes`` (25 MiB by
default) in parameter order; ``param.grad`` becomes a view into its bucket, so
nothing is copied before or after the allreduce, which runs in place with the
``1 / world_size`` scale fused into the reduction kernel.  Buckets are taken
from the communicator's symmetric memory when possible, which lets the switch
reduce them without staging.

For sharded optimizers (each rank updates 1/world_size of every bucket) the
same storage offers the two halves: :meth:`GradientBuckets.reduce_scatter`
leaves a rank with the reduced block it owns, :meth:`GradientBuckets.all_gather`
puts the blocks together again, both in place.

:meth:`GradientBuckets.overlap_with_backward` starts the allreduce of a bucket
as soon as autograd has produced all of its gradients, on a side stream, so
that the collectives of the late layers run while the early layers are still
in their backward pass; :meth:`GradientBuckets.finish` joins them."""
from __future__ import annotations

from typing import Iterable, Optional, Sequence

import torch

from .communicator import Communicator


def plan_buckets(numels: Sequence[int], elem_bytes: int, bucket_bytes: int) -> list[list[int]]:
    """Groups tensor indices into consecutive buckets of at most ``bucket_bytes``
    (a tensor larger than that gets a bucket of its own)."""
    buckets: list[list[int]] = []
    cur: list[int] = []
    cur_bytes = 0
    for i, n in enumerate(numels):
        b = n * elem_bytes
        if cur and cur_bytes + b > bucket_bytes:
            buckets.append(cur)
            cur, cur_bytes = [], 0
        cur.append(i)
        cur_bytes += b
    if cur:
        buckets.append(cur)
    return buckets


class GradientBuckets:
    """Flat gradient storage + bucketed allreduce.

    ``shapes``: one shape per gradient tensor.  ``comm`` may be ``None`` (or of
    world size 1) for single-process use; then :meth:`allreduce` only scales."""

    def __init__(self, shapes: Sequence[Sequence[int]], *, dtype=torch.float32, device="cuda",
                 comm: Optional[Communicator] = None, bucket_bytes: int = 25 << 20, symmetric: bool = True,
                 shardable: bool = False):
        self.comm = comm
        self.dtype = dtype
        self.shardable = shardable
        self.shapes = [tuple(s) for s in shapes]
        numels = [int(torch.Size(s).numel()) for s in self.shapes]
        esize = torch.empty((), dtype=dtype).element_size()
        # Every tensor starts on a 16-byte boundary inside its bucket.
        align = max(1, 16 // esize)
        self.plan = plan_buckets(numels, esize, bucket_bytes)
        self.flat: list[torch.Tensor] = []
        self.views: list[torch.Tensor] = [None] * len(self.shapes)  # type: ignore[list-item]
        for idxs in self.plan:
            offs, total = [], 0
            for i in idxs:
                offs.append(total)
                total += (numels[i] + align - 1) // align * align
            if shardable and comm is not None:
                # world_size equal blocks of whole 16-byte vectors
                unit = align * comm.world_size
                total = (total + unit - 1) // unit * unit
            if comm is not None and comm.world_size > 1 and symmetric:
                buf = comm.symmetric_empty(total, dtype)
            else:
                buf = torch.empty(total, dtype=dtype, device=device)
            buf.zero_()
            self.flat.append(buf)
            for i, o in zip(idxs, offs):
                self.views[i] = buf[o:o + numels[i]].view(self.shapes[i])

    @property
    def num_buckets(self) -> int:
        return len(self.flat)

    @property
    def nbytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self.flat)

    def attach(self, params: Iterable[torch.nn.Parameter]) -> None:
        """Makes every ``param.grad`` a view into the buckets."""
        for p, v in zip(params, self.views):
            p.grad = v

    def zero_(self) -> None:
        """Clears every bucket (the `zero_grad` of gradients that live here)."""
        torch._foreach_zero_(self.flat)

    def load(self, grads: Sequence[torch.Tensor]) -> None:
        """Copies gradients in (for callers that do not use :meth:`attach`)."""
        torch._foreach_copy_(list(self.views), list(grads))

    def allreduce(self, *, average: bool = True, wire=None, algo: str = "auto", sync: bool = False) -> None:
        """In-place sum (or mean) of every bucket over the ranks, on the current stream."""
        ws = 1 if self.comm is None else self.comm.world_size
        scale = 1.0 / ws if average else 1.0
        if self.comm is None:
            if scale != 1.0:
                torch._foreach_mul_(self.flat, scale)
            return
        for buf in self.flat:
            self.comm.allreduce(buf, algo=algo, scale=scale, wire=wire if buf.dtype == torch.float32 else None, sync=sync)

    def shards(self) -> list[torch.Tensor]:
        """This rank's block of every bucket (views; needs ``shardable=True``)."""
        if not self.shardable:
            raise ValueError("construct GradientBuckets with shardable=True")
        ws = 1 if self.comm is None else self.comm.world_size
        r = 0 if self.comm is None or ws == 1 else self.comm.rank
        out = []
        for buf in self.flat:
            m = buf.numel() // ws
            out.append(buf[r * m:(r + 1) * m])
        return out

    def reduce_scatter(self, *, average: bool = True, algo: str = "auto", sync: bool = False) -> list[torch.Tensor]:
        """Sum (or mean) over the ranks of this rank's block of every bucket, in place.

        Returns the blocks (the same views as :meth:`shards`); the rest of a bucket
        is left as it was."""
        mine = self.shards()
        ws = 1 if self.comm is None else self.comm.world_size
        scale = 1.0 / ws if average else 1.0
        if self.comm is None or ws == 1:
            if scale != 1.0:
                torch._foreach_mul_(mine, scale)
            return mine
        for buf, shard in zip(self.flat, mine):
            self.comm.reduce_scatter(buf, shard, algo=algo, scale=scale, sync=sync)
        return mine

    def all_gather(self, *, algo: str = "auto", sync: bool = False) -> None:
        """Every bucket = the ranks' blocks side by side (in place, from :meth:`shards`)."""
        mine = self.shards()
        if self.comm is None or self.comm.world_size == 1:
            return
        for buf, shard in zip(self.flat, mine):
            self.comm.all_gather(shard, buf, algo=algo, sync=sync)

    # ------------------------------------------------ overlap with backward
    def overlap_with_backward(self, params: Iterable[torch.nn.Parameter], *, average: bool = True, wire=None,
                              algo: str = "auto") -> None:
        """Attaches the gradients (see :meth:`attach`) and hooks every parameter: when the last gradient
        of a bucket has been accumulated, the bucket's allreduce is enqueued.

        Buckets start in descending order (autograd produces the last layers first) and a bucket waits
        for its turn, so every rank issues the same sequence of collectives.  On CUDA the collectives run
        on a stream of their own, behind the compute stream's work so far; :meth:`finish` makes the
        compute stream wait for them (call it before the optimizer reads the gradients).  For gradient
        accumulation, ``begin_step(communicate=False)`` before a backward pass that should only add up."""
        params = list(params)
        self.attach(params)
        self._ov = {"average": average, "wire": wire, "algo": algo, "stream": None, "communicate": True}
        self._bucket_of = {i: b for b, idxs in enumerate(self.plan) for i in idxs}
        # Gradients a bucket has to see before it may go; a bucket without trainable parameters never goes.
        self._expected = [sum(1 for i in idxs if params[i].requires_grad) for idxs in self.plan]
        self.remove_hooks()
        for i, p in enumerate(params):
            if p.requires_grad:
                self._handles.append(p.register_post_accumulate_grad_hook(self._make_hook(i)))
        self.begin_step()

    def begin_step(self, communicate: bool = True) -> None:
        """Resets the per-step bookkeeping (done by :meth:`finish` as well)."""
        self._ready = [0] * len(self.plan)
        self._next = len(self.plan) - 1
        self._ov["communicate"] = communicate

    def _make_hook(self, index: int):
        def hook(_param):
            if self._ov["communicate"]:
                self._ready[self._bucket_of[index]] += 1
                self._advance(force=False)
        return hook

    def _advance(self, force: bool) -> None:
        # Start every bucket whose turn has come: descending order, no gaps.
        while self._next >= 0:
            b = self._next
            if self._expected[b] > 0:
                if not force and self._ready[b] < self._expected[b]:
                    return
                self._start_bucket(b)
            self._next -= 1

    def _start_bucket(self, b: int) -> None:
        buf = self.flat[b]
        ws = 1 if self.comm is None else self.comm.world_size
        scale = 1.0 / ws if self._ov["average"] else 1.0
        if self.comm is None:
            if scale != 1.0:
                buf.mul_(scale)
            return
        if buf.is_cuda:
            if self._ov["stream"] is None:
                self._ov["stream"] = torch.cuda.Stream(device=buf.device)
            side = self._ov["stream"]
            side.wait_stream(torch.cuda.current_stream(buf.device))  # this bucket's gradients are complete
            self.comm.allreduce(buf, algo=self._ov["algo"], scale=scale,
                                wire=self._ov["wire"] if buf.dtype == torch.float32 else None, stream=side)
        else:
            self.comm.allreduce(buf, algo=self._ov["algo"], scale=scale)

    def finish(self) -> None:
        """Starts the buckets the hooks did not reach (parameters that took no part in this backward
        pass) and makes the current stream wait for all collectives of the step."""
        if not hasattr(self, "_ov"):
            raise ValueError("call overlap_with_backward first")
        if self._ov["communicate"]:
            self._advance(force=True)
        side = self._ov["stream"]
        if side is not None:
            torch.cuda.current_stream(side.device).wait_stream(side)
        self.begin_step(True)

    def remove_hooks(self) -> None:
        for h in getattr(self, "_handles", []):
            h.remove()
        self._handles = []
