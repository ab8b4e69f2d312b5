"""Worker of the multi-process host tests (CPU only): started by `ibcomm_run`,
uses the Python Communicator over the shared-memory transport.

    ibcomm_run -np N python tests/host_worker.py <case>
"""
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import numpy as np  # noqa: E402
import torch  # noqa: E402

import allreduce_proto_b200 as ar  # noqa: E402

RANK = int(os.environ.get("IBCOMM_RANK", "0"))
WS = int(os.environ.get("IBCOMM_WORLD_SIZE", "1"))


def case_allreduce(comm):
    # configs of the headline plumbing test: 4 Mi fp32 elements, uniform[-1, 1) seeded by rank
    n = 4_194_304
    x = torch.from_numpy(np.random.default_rng(RANK).uniform(-1, 1, n).astype(np.float32))
    want = np.zeros(n, dtype=np.float64)
    for r in range(WS):
        want += np.random.default_rng(r).uniform(-1, 1, n).astype(np.float32).astype(np.float64)
    for algo in ("ring", "rabenseifner"):
        y = torch.empty_like(x)
        comm.allreduce(x, y, algo=algo)
        if not np.allclose(y.numpy().astype(np.float64), want, rtol=1e-5, atol=1e-5):
            print(f"rank {RANK}: {algo} mismatch", file=sys.stderr)
            return 1
    z = torch.arange(1000, dtype=torch.int64) + RANK
    comm.allreduce(z, algo="ring")
    if not torch.equal(z, torch.arange(1000, dtype=torch.int64) * WS + WS * (WS - 1) // 2):
        return 1
    d = torch.full((777,), 0.5 * (RANK + 1), dtype=torch.float64)
    comm.allreduce(d, algo="rabenseifner", scale=2.0)
    return 0 if torch.allclose(d, torch.full((777,), float(WS * (WS + 1) / 2), dtype=torch.float64)) else 1


def case_rsag(comm):
    # Reduce-scatter and all-gather on host buffers: block r belongs to rank r.
    for m in (1, 1000, 1_500_001):  # the last one is larger than a transport ring
        n = m * WS
        x = torch.from_numpy(np.random.default_rng(100 + RANK).integers(-1000, 1000, n).astype(np.int64))
        want = np.zeros(n, dtype=np.int64)
        for r in range(WS):
            want += np.random.default_rng(100 + r).integers(-1000, 1000, n).astype(np.int64)
        y = torch.zeros(m, dtype=torch.int64)
        comm.reduce_scatter(x, y)
        if not np.array_equal(y.numpy(), want[RANK * m:(RANK + 1) * m]):
            print(f"rank {RANK}: reduce_scatter m={m} mismatch", file=sys.stderr)
            return 1
        z = torch.zeros(n, dtype=torch.int64)
        comm.all_gather(y, z)
        if not np.array_equal(z.numpy(), want):
            print(f"rank {RANK}: all_gather m={m} mismatch", file=sys.stderr)
            return 1
        # in place, float, with the scale
        f = x.to(torch.float64)
        mine = f[RANK * m:(RANK + 1) * m]
        comm.reduce_scatter(f, mine, scale=0.5)
        comm.all_gather(mine, f)
        if not np.allclose(f.numpy(), want * 0.5):
            print(f"rank {RANK}: in-place reduce_scatter + all_gather m={m} mismatch", file=sys.stderr)
            return 1
    return 0


def case_sharded_buckets(comm):
    # Gradient buckets on host tensors: reduce-scatter leaves a rank its block
    # of the mean, all-gather rebuilds the whole; the result equals the allreduce.
    shapes = [(64, 3, 7, 7), (64,), (1000, 33), (5,), (12345,)]
    def grads(r):
        g = torch.Generator().manual_seed(r)
        return [torch.rand(s, generator=g) * 2 - 1 for s in shapes]
    want = [sum(gs) / WS for gs in zip(*[grads(r) for r in range(WS)])]
    b = ar.GradientBuckets(shapes, device="cpu", comm=comm, bucket_bytes=64 << 10, symmetric=False, shardable=True)
    b.load(grads(RANK))
    mine = b.reduce_scatter(average=True)
    if len(mine) != b.num_buckets or any(s.numel() * WS != f.numel() for s, f in zip(mine, b.flat)):
        return 1
    b.all_gather()
    for v, w in zip(b.views, want):
        if not torch.allclose(v, w, rtol=1e-5, atol=1e-6):
            print(f"rank {RANK}: sharded buckets mismatch", file=sys.stderr)
            return 1
    ref = ar.GradientBuckets(shapes, device="cpu", comm=comm, bucket_bytes=64 << 10, symmetric=False)
    ref.load(grads(RANK))
    ref.allreduce(average=True, sync=True)
    for v, w in zip(ref.views, want):
        if not torch.allclose(v, w, rtol=1e-5, atol=1e-6):
            print(f"rank {RANK}: bucket allreduce mismatch", file=sys.stderr)
            return 1
    return 0


def case_messaging(comm):
    to, frm = (RANK + 1) % WS, (RANK - 1) % WS
    out = np.arange(100000, dtype=np.int32) + RANK
    inn = np.zeros_like(out)
    comm.send(to, out, blocking=False)
    comm.recv(frm, inn, blocking=False)
    while not comm.recv_poll(frm):
        pass
    comm.send_wait(to)
    if not np.array_equal(inn, np.arange(100000, dtype=np.int32) + frm):
        return 1
    b = np.full(33, RANK, dtype=np.int64)
    comm.bcast(b, root=1 % WS)
    comm.barrier()
    return 0 if np.all(b == 1 % WS) else 1


def case_peer_exit(comm):
    """The last rank exits without taking part; the others must fail with the
    transport error code instead of hanging."""
    if RANK == WS - 1:
        return 0
    comm.set_timeout_ms(1500)
    x = torch.ones(1 << 16)
    t0 = time.time()
    try:
        comm.allreduce(x, algo="ring")
    except ar.IbcommError as e:
        return 0 if e.code == ar.TRANSPORT_ERROR and time.time() - t0 < 20 else 1
    return 1


def case_shrink(comm):
    """The last rank leaves between steps; the others see the transport error on their next
    collective, form a smaller communicator and carry on."""
    x = torch.full((1 << 12,), float(RANK + 1))
    comm.allreduce(x, algo="ring")                       # step 1: everybody
    if not torch.allclose(x, torch.full_like(x, WS * (WS + 1) / 2)):
        return 1
    comm.barrier()
    if RANK == WS - 1:
        comm.close()
        return 0                                          # leaves with nothing in flight
    comm.set_timeout_ms(1500)
    y = torch.ones(1 << 12)
    try:
        comm.allreduce(y, algo="ring")                   # step 2: one rank is missing
        return 1
    except ar.IbcommError as e:
        if e.code != ar.TRANSPORT_ERROR:
            return 1
    comm.close()
    survivors = list(range(WS - 1))
    small = ar.Communicator.from_env(tag="after_failure", ranks=survivors)
    z = torch.full((1 << 12,), float(RANK + 1))
    small.allreduce(z, algo="rabenseifner")
    ok = small.world_size == WS - 1 and torch.allclose(z, torch.full_like(z, (WS - 1) * WS / 2))
    small.close()
    return 0 if ok else 1


def case_trace(comm):
    comm.set_timer_base()
    x = torch.ones(1 << 12)
    comm.allreduce(x)
    comm.dump_trace()
    return 0


def main():
    case = sys.argv[1]
    comm = ar.Communicator.from_env()
    rc = globals()[f"case_{case}"](comm)
    if case not in ("peer_exit", "shrink"):   # these end with ranks that are gone
        comm.barrier()
    comm.close()
    return rc


if __name__ == "__main__":
    sys.exit(main())
