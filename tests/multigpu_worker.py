"""Worker of the multi-GPU tests: one process per GPU, started by `ibcomm_run`
(which sets IBCOMM_RANK / IBCOMM_WORLD_SIZE / IBCOMM_BOOTSTRAP_DIR).

    ibcomm_run -np N python tests/multigpu_worker.py <case>

Exit status 0 = the case passed on this rank."""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402

import allreduce_proto_b200 as ar  # noqa: E402

RANK = int(os.environ.get("IBCOMM_RANK", "0"))
WS = int(os.environ.get("IBCOMM_WORLD_SIZE", "1"))


def seeded(n, dtype, r, seed=0):
    g = torch.Generator(device="cuda")
    g.manual_seed(1000 * seed + r)
    if dtype in (torch.int32, torch.int64):
        return torch.randint(-1000, 1000, (n,), device="cuda", dtype=dtype, generator=g)
    return (torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dtype)


def expected(n, dtype, scale, seed=0):
    acc = torch.zeros(n, dtype=torch.float64, device="cuda")
    for r in range(WS):
        acc += seeded(n, dtype, r, seed).double()
    return acc * scale


def close(out, want, dtype, wire=None):
    if dtype in (torch.int32, torch.int64):
        return torch.equal(out.double(), want)
    if dtype == torch.float64:
        tol = 1e-12
    elif dtype == torch.float32 and wire is None:
        tol = 1e-6 * WS
    else:
        tol = 2e-2 * WS
    return torch.allclose(out.double(), want, rtol=tol, atol=tol)


def case_allreduce(comm):
    info = comm.device_info(connect=True)
    algos = ["ring", "rabenseifner", "oneshot", "direct", "auto"] + (["nvls"] if info["nvls"] else [])
    for algo in algos:
        for dtype in (torch.float32, torch.bfloat16, torch.int32):
            if algo == "nvls" and dtype == torch.int32:
                continue
            for n in (WS, 1000, 65536, (1 << 20) + 5, 8 << 20):
                if algo == "oneshot" and n * torch.empty((), dtype=dtype).element_size() > (512 << 10):
                    continue
                scale = 1.0 if dtype == torch.int32 else 0.5
                x = seeded(n, dtype, RANK, seed=n % 97)
                y = torch.empty_like(x)
                comm.allreduce(x, y, algo=algo, scale=scale, sync=True)
                if not close(y, expected(n, dtype, scale, seed=n % 97), dtype):
                    print(f"rank {RANK}: {algo} {dtype} n={n} mismatch", file=sys.stderr)
                    return 1
    # in place + wire compression
    x = seeded(1 << 20, torch.float32, RANK, seed=5)
    comm.allreduce(x, algo="ring", wire=torch.bfloat16, sync=True)
    if not close(x, expected(1 << 20, torch.float32, 1.0, seed=5), torch.float32, wire=torch.bfloat16):
        return 1
    return 0


def case_staged(comm):
    """Ordinary buffers over several pool windows; the odd lengths end in a short last window."""
    info = comm.device_info(connect=True)
    rc = 0
    for algo in ["direct"] + (["nvls"] if info["nvls"] else []):
        for n in ((8 << 20) + 3, 40_000_001, 17_000_005):
            x = seeded(n, torch.float32, RANK, seed=3)
            y = torch.empty_like(x)
            comm.allreduce(x, y, algo=algo, scale=0.5, sync=True)
            if not close(y, expected(n, torch.float32, 0.5, seed=3), torch.float32):
                bad = ((y.double() - expected(n, torch.float32, 0.5, seed=3)).abs() > 1e-4).nonzero().flatten()
                print(f"rank {RANK}: staged {algo} n={n} mismatch: {bad.numel()} elements, first {bad[:4].tolist()}, last {bad[-2:].tolist()}", file=sys.stderr)
                rc = 1
            comm.allreduce(x, algo=algo, sync=True)  # in place
            if not close(x, expected(n, torch.float32, 1.0, seed=3), torch.float32):
                bad = ((x.double() - expected(n, torch.float32, 1.0, seed=3)).abs() > 1e-4).nonzero().flatten()
                print(f"rank {RANK}: staged in-place {algo} n={n} mismatch: {bad.numel()} elements, first {bad[:4].tolist()}, last {bad[-2:].tolist()}", file=sys.stderr)
                rc = 1
    return rc


def case_symmetric(comm):
    """Zero-copy buffers: symmetric memory, switch reduction when available."""
    n = (4 << 20) + 3
    a = comm.symmetric_empty(n, torch.float32)
    b = comm.symmetric_empty(n, torch.float32)
    for it in range(3):
        a.copy_(seeded(n, torch.float32, RANK, seed=it))
        comm.allreduce(a, b, scale=1.0 / WS, sync=True)
        if not close(b, expected(n, torch.float32, 1.0 / WS, seed=it), torch.float32):
            print(f"rank {RANK}: symmetric out-of-place mismatch", file=sys.stderr)
            return 1
        comm.allreduce(a, scale=1.0 / WS, sync=True)  # in place
        if not close(a, expected(n, torch.float32, 1.0 / WS, seed=it), torch.float32):
            print(f"rank {RANK}: symmetric in-place mismatch", file=sys.stderr)
            return 1
    h = comm.symmetric_empty(1 << 20, torch.bfloat16)
    h.copy_(seeded(1 << 20, torch.bfloat16, RANK, seed=9))
    comm.allreduce(h, sync=True)
    if not close(h, expected(1 << 20, torch.bfloat16, 1.0, seed=9), torch.bfloat16):
        return 1
    return 0


def case_registered(comm):
    """Ordinary torch tensors mapped into the peers (CUDA IPC): direct two-shot without staging."""
    rc = 0
    # Ranks allocate differently first, so that the tensors sit at different
    # offsets of their allocations on different ranks.
    pad = torch.empty(1000 * (RANK + 1), device="cuda")
    for n in (1000, (4 << 20) + 4):
        x = torch.empty(n, device="cuda")
        y = torch.empty(n, device="cuda")
        rx, ry = comm.register(x), comm.register(y)
        if rx < 0 or ry < 0:
            print(f"rank {RANK}: registration not available", file=sys.stderr)
            return 1
        for it in range(2):
            x.copy_(seeded(n, torch.float32, RANK, seed=it))
            comm.allreduce(x, y, scale=1.0 / WS, sync=True)
            algo = comm.device_info()["last_algo"]
            if n > (1 << 20) and algo != "direct":
                print(f"rank {RANK}: registered buffers ran {algo}", file=sys.stderr)
                rc = 1
            if not close(y, expected(n, torch.float32, 1.0 / WS, seed=it), torch.float32):
                print(f"rank {RANK}: registered out-of-place n={n} mismatch", file=sys.stderr)
                rc = 1
            # A slice at an odd element (not 16-byte aligned): staged on every rank alike.
            comm.allreduce(x[1:], y[1:], algo="direct", sync=True)
            if not close(y[1:], expected(n, torch.float32, 1.0, seed=it)[1:], torch.float32):
                print(f"rank {RANK}: registered odd slice n={n} mismatch", file=sys.stderr)
                rc = 1
            # An aligned slice, in place.
            comm.allreduce(x[4:], algo="direct", sync=True)
            if not close(x[4:], expected(n, torch.float32, 1.0, seed=it)[4:], torch.float32):
                print(f"rank {RANK}: registered in-place slice n={n} mismatch", file=sys.stderr)
                rc = 1
        comm.deregister(rx)
        comm.deregister(ry)
        # Without the registration the same tensors go through the pool again.
        x.copy_(seeded(n, torch.float32, RANK, seed=7))
        comm.allreduce(x, y, sync=True)
        if not close(y, expected(n, torch.float32, 1.0, seed=7), torch.float32):
            print(f"rank {RANK}: after deregistration n={n} mismatch", file=sys.stderr)
            rc = 1
    del pad
    return rc


def case_registered_switch(comm):
    """Ordinary torch tensors that registration binds to the NVSwitch multicast: the switch kernel reduces and
    broadcasts them in place.  Large tensors get allocations of their own, so they start on a granule on every
    rank; where the box or the driver cannot bind them the registration stays peer-mapped and the case only
    checks the results."""
    info = comm.device_info(connect=True)
    rc = 0
    n = 12 << 20  # 48 MiB: an allocation of its own in the caching allocator
    x = torch.empty(n, device="cuda")
    y = torch.empty(n, device="cuda")
    rx, ry = comm.register(x), comm.register(y)
    if rx < 0 or ry < 0:
        print(f"rank {RANK}: registration not available", file=sys.stderr)
        return 1
    bound = comm.device_info()["switch_registrations"]
    if RANK == 0:
        print(f"switch registrations: {bound} (nvls {info['nvls']})")
    if info["nvls"] and bound not in (0, 2):
        print(f"rank {RANK}: {bound} of 2 registrations bound to the switch", file=sys.stderr)
        rc = 1
    algos = ["auto", "direct"] + (["nvls"] if info["nvls"] else [])
    for it, algo in enumerate(algos):
        x.copy_(seeded(n, torch.float32, RANK, seed=it))
        comm.allreduce(x, y, algo=algo, scale=1.0 / WS, sync=True)
        used = comm.device_info()["last_algo"]
        if algo == "auto" and bound == 2 and WS > 2 and used != "nvls":
            print(f"rank {RANK}: switch-bound registered buffers ran {used}", file=sys.stderr)
            rc = 1
        if not close(y, expected(n, torch.float32, 1.0 / WS, seed=it), torch.float32):
            print(f"rank {RANK}: registered ({algo}) mismatch", file=sys.stderr)
            rc = 1
        # in place on an aligned slice, and a sub-range of both buffers
        comm.allreduce(x[1 << 20:], algo=algo, sync=True)
        if not close(x[1 << 20:], expected(n, torch.float32, 1.0, seed=it)[1 << 20:], torch.float32):
            print(f"rank {RANK}: registered in-place slice ({algo}) mismatch", file=sys.stderr)
            rc = 1
    comm.deregister(rx)
    comm.deregister(ry)
    if comm.device_info()["switch_registrations"] != 0:
        print(f"rank {RANK}: registrations left bound after deregister", file=sys.stderr)
        rc = 1
    x.copy_(seeded(n, torch.float32, RANK, seed=9))
    comm.allreduce(x, y, sync=True)
    if not close(y, expected(n, torch.float32, 1.0, seed=9), torch.float32):
        print(f"rank {RANK}: after deregistration mismatch", file=sys.stderr)
        rc = 1
    return rc


def case_rsag(comm):
    """Reduce-scatter and all-gather: ordinary, registered and symmetric buffers; every algorithm the box has."""
    rc = 0
    info = comm.device_info(connect=True)
    algos = ["auto", "direct"] + (["nvls"] if info["nvls"] else [])
    for m in (4, 1000, (1 << 20) + 8, 3_000_001):
        x = seeded(m * WS, torch.float32, RANK, seed=m)
        want = expected(m * WS, torch.float32, 0.5, seed=m)
        for algo in algos:
            if algo == "nvls" and (m * 4) % 16 != 0:
                continue
            y = torch.zeros(m, device="cuda")
            comm.reduce_scatter(x, y, algo=algo, scale=0.5, sync=True)
            if not close(y, want[RANK * m:(RANK + 1) * m], torch.float32):
                print(f"rank {RANK}: reduce_scatter {algo} m={m} mismatch", file=sys.stderr)
                rc = 1
            z = torch.zeros(m * WS, device="cuda")
            comm.all_gather(y, z, algo=algo, sync=True)
            if not close(z, want, torch.float32):
                print(f"rank {RANK}: all_gather {algo} m={m} mismatch", file=sys.stderr)
                rc = 1
    # Zero-copy: symmetric memory (switch path where available) and registered tensors (direct).
    m = (1 << 20) + 16
    sx = comm.symmetric_empty(m * WS, torch.float32)
    sz = comm.symmetric_empty(m * WS, torch.float32)
    rx = torch.empty(m * WS, device="cuda")
    rz = torch.empty(m * WS, device="cuda")
    ids = [comm.register(rx), comm.register(rz)]
    for name, bx, bz in (("symmetric", sx, sz), ("registered", rx, rz)):
        for it in range(2):
            bx.copy_(seeded(m * WS, torch.float32, RANK, seed=it + 50))
            want = expected(m * WS, torch.float32, 1.0, seed=it + 50)
            y = torch.zeros(m, device="cuda")
            comm.reduce_scatter(bx, y, sync=True)
            if not close(y, want[RANK * m:(RANK + 1) * m], torch.float32):
                print(f"rank {RANK}: {name} reduce_scatter mismatch ({comm.device_info()['last_algo']})", file=sys.stderr)
                rc = 1
            comm.all_gather(y, bz, sync=True)
            if not close(bz, want, torch.float32):
                print(f"rank {RANK}: {name} all_gather mismatch ({comm.device_info()['last_algo']})", file=sys.stderr)
                rc = 1
            # in place: my block of the input is the output, then gathered in place
            mine = bx[RANK * m:(RANK + 1) * m]
            comm.reduce_scatter(bx, mine, sync=True)
            comm.all_gather(mine, bx, sync=True)
            if not close(bx, want, torch.float32):
                print(f"rank {RANK}: {name} in-place reduce_scatter + all_gather mismatch", file=sys.stderr)
                rc = 1
    for rid in ids:
        if rid >= 0:
            comm.deregister(rid)
    return rc


def case_sendrecv(comm):
    """Device buffers through the mailbox kernels; ring of neighbours plus a broadcast."""
    comm.device_info(connect=True)
    to, frm = (RANK + 1) % WS, (RANK - 1) % WS
    for nbytes in (0, 4, 1000, 256 << 10, (3 << 20) + 17, (40 << 20) + 48):
        # Payload: a byte pattern that depends on the position and on the sender; compared in full.
        pos = torch.arange(nbytes, device="cuda", dtype=torch.int64)
        out = ((pos * 7 + RANK * 13) % 251).to(torch.uint8)
        inn = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        comm.send(to, out, blocking=False)
        comm.recv(frm, inn, blocking=True)
        comm.send_wait(to)
        if not torch.equal(inn, ((pos * 7 + frm * 13) % 251).to(torch.uint8)):
            bad = (inn != ((pos * 7 + frm * 13) % 251).to(torch.uint8)).nonzero().flatten()
            print(f"rank {RANK}: sendrecv {nbytes} mismatch at {bad[:4].tolist()} ({bad.numel()} bytes)", file=sys.stderr)
            return 1
    # an odd (only byte-aligned) view takes the byte path
    base_o = torch.arange(100001, device="cuda", dtype=torch.int64).remainder(199).to(torch.uint8)
    base_i = torch.zeros(100003, dtype=torch.uint8, device="cuda")
    comm.send(to, base_o[1:], blocking=False)
    comm.recv(frm, base_i[3:], blocking=True)
    comm.send_wait(to)
    if not torch.equal(base_i[3:], base_o[1:]):
        print(f"rank {RANK}: unaligned sendrecv mismatch", file=sys.stderr)
        return 1
    # Broadcasts: through the switch where the box has multicast (lengths that are multiples of 16, several
    # slots' worth, changing roots so that every rank's slot credits are exercised), by sends otherwise
    # (a length that is not a multiple of 16) - and from a buffer that is only byte-aligned.
    for it, (nbytes, root) in enumerate(((16384, WS - 1), (20 << 20, 0), (20 << 20, WS - 1), (1 << 20, 1 % WS), (1000, 0), (48 << 20, 0))):
        pos = torch.arange(nbytes, device="cuda", dtype=torch.int64)
        want = ((pos * 3 + root * 17 + it) % 253).to(torch.uint8)
        t = want.clone() if RANK == root else torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        comm.bcast(t, root=root)
        if not torch.equal(t, want):
            print(f"rank {RANK}: bcast {nbytes} from {root} mismatch", file=sys.stderr)
            return 1
    base = torch.zeros(4096 + 1, dtype=torch.uint8, device="cuda")
    view = base[1:]
    if RANK == 0:
        view.copy_(torch.arange(4096, device="cuda").remainder(101).to(torch.uint8))
    comm.bcast(view, root=0)
    if not torch.equal(view, torch.arange(4096, device="cuda").remainder(101).to(torch.uint8)):
        print(f"rank {RANK}: unaligned bcast mismatch", file=sys.stderr)
        return 1
    # host buffers still travel over the host transport
    hs = torch.full((1000,), float(RANK))
    hr = torch.zeros(1000)
    comm.send(to, hs, blocking=False)
    comm.recv(frm, hr, blocking=True)
    comm.send_wait(to)
    return 0 if torch.all(hr == float(frm)) else 1


def case_buckets(comm):
    from allreduce_proto_b200.models import resnet50_param_shapes, synthetic_grads
    shapes = [s for _, s in resnet50_param_shapes()]
    for dtype, wire in ((torch.float32, None), (torch.float32, torch.bfloat16), (torch.bfloat16, None)):
        buckets = ar.GradientBuckets(shapes, dtype=dtype, comm=comm, bucket_bytes=25 << 20)
        grads = synthetic_grads("cuda", dtype=dtype, seed=RANK)
        buckets.load(grads)
        buckets.allreduce(average=True, wire=wire, sync=True)
        want = [torch.zeros(s, dtype=torch.float64, device="cuda") for s in shapes]
        for r in range(WS):
            for w, g in zip(want, synthetic_grads("cuda", dtype=dtype, seed=r)):
                w += g.double()
        tol = 1e-7 if (dtype == torch.float32 and wire is None) else 3e-5
        for v, w in zip(buckets.views, want):
            if not torch.allclose(v.double(), w / WS, rtol=2e-2 if tol > 1e-6 else 1e-5, atol=tol):
                print(f"rank {RANK}: bucket mismatch {dtype} wire={wire}", file=sys.stderr)
                return 1
    return 0


def case_sharded_buckets(comm):
    """ResNet-50 gradients in shardable buckets: reduce-scatter (mean), then all-gather, equals the allreduce."""
    from allreduce_proto_b200.models import resnet50_param_shapes, synthetic_grads
    shapes = [s for _, s in resnet50_param_shapes()]
    buckets = ar.GradientBuckets(shapes, comm=comm, bucket_bytes=25 << 20, shardable=True)
    buckets.load(synthetic_grads("cuda", seed=RANK))
    mine = buckets.reduce_scatter(average=True, sync=True)
    if any(s.numel() * WS != f.numel() for s, f in zip(mine, buckets.flat)):
        return 1
    buckets.all_gather(sync=True)
    want = [torch.zeros(s, dtype=torch.float64, device="cuda") for s in shapes]
    for r in range(WS):
        for w, g in zip(want, synthetic_grads("cuda", seed=r)):
            w += g.double()
    for v, w in zip(buckets.views, want):
        if not torch.allclose(v.double(), w / WS, rtol=1e-5, atol=1e-7):
            print(f"rank {RANK}: sharded bucket mismatch", file=sys.stderr)
            return 1
    return 0


def case_graph(comm):
    """Collectives captured in a CUDA graph and replayed: the kernels take their
    call number from device memory, so a replay is a new, correctly sequenced call."""
    info = comm.device_info(connect=True)
    n = 1 << 16
    cases = [("oneshot", n), ("ring", 1 << 20), ("rabenseifner", 1 << 20), ("direct", 1 << 20)]
    if info["nvls"]:
        cases.append(("nvls", 1 << 20))
    stream = torch.cuda.Stream()
    for algo, m in cases:
        x = comm.symmetric_empty(m, torch.float32)
        y = comm.symmetric_empty(m, torch.float32)
        x.copy_(seeded(m, torch.float32, RANK, seed=1))
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            # warm-up: every distinct call is issued once outside the capture,
            # which builds and uploads its program (an allocation)
            comm.allreduce(x, y, algo=algo, scale=0.5)
            comm.allreduce(y, x, algo=algo, scale=1.0)
        stream.synchronize()
        x.copy_(seeded(m, torch.float32, RANK, seed=1))
        comm.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            comm.allreduce(x, y, algo=algo, scale=0.5)
            comm.allreduce(y, x, algo=algo, scale=1.0)  # two dependent collectives per replay
        for it in range(4):
            x.copy_(seeded(m, torch.float32, RANK, seed=10 + it))
            torch.cuda.synchronize()
            comm.barrier()
            g.replay()
            torch.cuda.synchronize()
            comm.check()
            want = expected(m, torch.float32, 0.5, seed=10 + it) * WS
            if not torch.allclose(x.double(), want, rtol=1e-5 * WS, atol=1e-5 * WS):
                print(f"rank {RANK}: graph replay {it} of {algo} mismatch", file=sys.stderr)
                return 1
        # an ordinary call after the replays still lines up with the peers
        comm.allreduce(x, y, algo=algo, sync=True)
    return 0


def case_trace(comm):
    """Device-side trace: per-op %globaltimer stamps end up in the trace file."""
    comm.set_timer_base()
    x = seeded(1 << 20, torch.float32, RANK)
    for algo in ("ring", "rabenseifner"):
        comm.allreduce(x.clone(), algo=algo, sync=True)
    # The pipelined staged kernel stamps per role and window: an ordinary tensor of three windows
    # (the staging is cut to 1 MiB windows for this), then the stamps must tell the story in order.
    ar.utils.set_tunable("IBCOMM_STAGED_WINDOW_KIB", 1024)
    y = seeded(3 << 18, torch.float32, RANK)
    comm.allreduce(y, algo="direct", sync=True)
    ar.utils.set_tunable("IBCOMM_STAGED_WINDOW_KIB", -1)
    t = comm.staged_timeline()
    rc = 0
    if t["windows"] != 3:
        print(f"rank {RANK}: staged timeline has {t['windows']} windows, expected 3", file=sys.stderr)
        rc = 1
    for k in range(t["windows"]):
        start, stored, published = t["reduce"][k]
        # (a role stamps after it has published, so the next role's stamp may come a moment earlier)
        if not (t["load"][k][1] <= start + 5.0 and start <= stored <= published and published <= t["store"][k][0] + 5.0
                and t["store"][k][0] <= t["store"][k][1]):
            print(f"rank {RANK}: staged timeline out of order at window {k}: {t}", file=sys.stderr)
            rc = 1
    comm.dump_trace()
    return rc


def case_leave(comm):
    """Failure detection without faulting a GPU: after one good allreduce the
    last rank leaves between steps; the others' next collective runs into its
    wait limit, returns error code 2 and leaves the context usable."""
    x = torch.ones(1 << 16, device="cuda")
    comm.allreduce(x, algo="ring", sync=True)
    if not torch.all(x == float(WS)):
        return 1
    if RANK == WS - 1:
        torch.cuda.synchronize()
        return 0
    comm.set_timeout_ms(1000)
    try:
        comm.allreduce(x, algo="ring", sync=True)
    except ar.IbcommError as e:
        ok = e.code == ar.TRANSPORT_ERROR
        y = torch.ones(16, device="cuda") * 2  # the context still works
        return 0 if ok and float(y.sum()) == 32.0 else 1
    return 1


def case_pipelined(comm):
    """Ordinary (unmapped) buffers through the pipelined staged kernel: lengths of one and of many
    windows, both copy modes, in place, and fp32 with a 16-bit wire (which every rank must round alike)."""
    info = comm.device_info(connect=True)
    rc = 0
    algos = ["direct"] + (["nvls"] if info["nvls"] else [])
    for algo in algos:
        for tma in (1, 0):
            ar.utils.set_tunable("IBCOMM_STAGED_TMA", tma)
            for n in (4 * WS, 1 << 16, 8 << 20, 40_000_000):
                x = seeded(n, torch.float32, RANK, seed=3)
                y = torch.empty_like(x)
                comm.allreduce(x, y, algo=algo, scale=0.5, sync=True)
                if not close(y, expected(n, torch.float32, 0.5, seed=3), torch.float32):
                    print(f"rank {RANK}: pipelined {algo} tma={tma} n={n} mismatch", file=sys.stderr)
                    rc = 1
            x = seeded(20_000_000, torch.float32, RANK, seed=4)
            for _ in range(3):  # back to back, no host synchronisation in between
                comm.allreduce(x, algo=algo, scale=1.0 / WS)
            torch.cuda.synchronize()
            comm.check()
            want = expected(20_000_000, torch.float32, 1.0 / WS, seed=4)  # the mean of equal values is the value
            if not close(x, want, torch.float32):
                print(f"rank {RANK}: pipelined in-place {algo} tma={tma} mismatch", file=sys.stderr)
                rc = 1
        ar.utils.set_tunable("IBCOMM_STAGED_TMA", -1)
        for wire in (torch.bfloat16, torch.float16):
            n = 10_000_000
            x = seeded(n, torch.float32, RANK, seed=8)
            y = torch.empty_like(x)
            comm.allreduce(x, y, algo=algo, wire=wire, scale=1.0 / WS, sync=True)
            if not close(y, expected(n, torch.float32, 1.0 / WS, seed=8), torch.float32, wire=wire):
                print(f"rank {RANK}: {algo} with {wire} wire mismatch", file=sys.stderr)
                rc = 1
            # all ranks hold the same bits
            digest = y.view(torch.int32).sum(dtype=torch.int64).reshape(1).double().repeat(8)
            total = digest.clone()
            comm.allreduce(total, algo="oneshot", sync=True)
            if abs(float(total[0].item()) - WS * float(digest[0].item())) > 0.5:
                print(f"rank {RANK}: {algo} with {wire} wire: ranks differ", file=sys.stderr)
                rc = 1
    return rc


def case_hybrid(comm):
    """The hybrid two-shot (part of the message reduced in the switch, the rest by peer loads, in one kernel)."""
    info = comm.device_info(connect=True)
    if not info["nvls"]:
        return 0
    rc = 0
    n = (16 << 20) + 5
    a = comm.symmetric_empty(n, torch.float32)
    b = comm.symmetric_empty(n, torch.float32)
    try:
        for pct, sw, di in ((25, 48, 96), (10, 96, 16), (90, 8, 100), (50, 1, 1)):
            ar.utils.set_tunable("IBCOMM_NVLS_HYBRID", pct)
            ar.utils.set_tunable("IBCOMM_NVLS_HYBRID_SWITCH_CTAS", sw)
            ar.utils.set_tunable("IBCOMM_NVLS_HYBRID_DIRECT_CTAS", di)
            for it in range(2):
                a.copy_(seeded(n, torch.float32, RANK, seed=it + pct))
                comm.allreduce(a, b, algo="nvls", scale=1.0 / WS, sync=True)
                if comm.device_info()["last_channels"] != sw + di:
                    print(f"rank {RANK}: the hybrid kernel did not run ({comm.device_info()})", file=sys.stderr)
                    rc = 1
                if not close(b, expected(n, torch.float32, 1.0 / WS, seed=it + pct), torch.float32):
                    print(f"rank {RANK}: hybrid {pct}% out-of-place mismatch", file=sys.stderr)
                    rc = 1
                comm.allreduce(a, algo="nvls", sync=True)  # in place
                if not close(a, expected(n, torch.float32, 1.0, seed=it + pct), torch.float32):
                    print(f"rank {RANK}: hybrid {pct}% in-place mismatch", file=sys.stderr)
                    rc = 1
    finally:
        for k in ("IBCOMM_NVLS_HYBRID", "IBCOMM_NVLS_HYBRID_SWITCH_CTAS", "IBCOMM_NVLS_HYBRID_DIRECT_CTAS"):
            ar.utils.set_tunable(k, -1)
    return rc


def case_p2p_errors(comm):
    """Device Send/Recv failure paths on two ranks; nothing faults, every wait is bounded."""
    comm.device_info(connect=True)
    other = 1 - RANK
    # (1) a receive without a matching send runs out of time on rank 1 ...
    if RANK == 1:
        comm.set_timeout_ms(500)
        buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
        try:
            comm.recv(0, buf, blocking=True)
            print("rank 1: the unmatched receive returned", file=sys.stderr)
            return 1
        except ar.IbcommError as e:
            if e.code != ar.TRANSPORT_ERROR:
                return 1
        comm.set_timeout_ms(10000)
    comm.barrier()
    # ... and the other direction (its own counters) still works afterwards.
    out = torch.full((1 << 20,), 7 + RANK, dtype=torch.uint8, device="cuda")
    inn = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    if RANK == 1:
        comm.send(0, out, blocking=True)
    else:
        comm.recv(1, inn, blocking=True)
        if not torch.all(inn == 8):
            print("rank 0: message after the timed-out receive is wrong", file=sys.stderr)
            return 1
    comm.barrier()
    # (2) length mismatch: 1000 bytes sent, 2000 expected.
    if RANK == 1:
        comm.send(0, out[:1000], blocking=True)
    else:
        try:
            comm.recv(1, inn[:2000], blocking=True)
            print("rank 0: the mismatched receive returned", file=sys.stderr)
            return 1
        except ar.IbcommError as e:
            if e.code != ar.TRANSPORT_ERROR or "length mismatch" not in str(e):
                print(f"rank 0: unexpected error {e}", file=sys.stderr)
                return 1
    comm.barrier()
    # (3) both sides counted one piece for that message, so the next one lines up.
    if RANK == 1:
        comm.send(0, out[:5000], blocking=True)
    else:
        comm.recv(1, inn[:5000], blocking=True)
        if not torch.all(inn[:5000] == 8):
            return 1
    return 0


def case_overlap(comm):
    """Collectives on a side stream next to a compute stream that is kept busy."""
    import time
    comm.device_info(connect=True)
    n = 8 << 20
    side = torch.cuda.Stream()
    a = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
    xs = [seeded(n, torch.float32, RANK, seed=s) for s in range(4)]
    ys = [torch.empty_like(x) for x in xs]
    sym = comm.symmetric_empty(n, torch.float32)
    sym.copy_(xs[0])
    torch.cuda.synchronize()
    comm.barrier()
    t0 = time.time()
    for rep in range(3):
        for _ in range(40):
            a @ a  # compute stream: a few hundred microseconds each
        with torch.cuda.stream(side):
            for i, algo in enumerate(("ring", "rabenseifner", "direct", "auto")):
                comm.allreduce(xs[i], ys[i], algo=algo, scale=1.0 / WS, stream=side)
            comm.allreduce(sym, algo="auto", scale=1.0, stream=side)
        for _ in range(40):
            a @ a
    torch.cuda.synchronize()
    elapsed = time.time() - t0
    comm.check()
    for i in range(4):
        if not close(ys[i], expected(n, torch.float32, 1.0 / WS, seed=i), torch.float32):
            print(f"rank {RANK}: overlap result {i} mismatch", file=sys.stderr)
            return 1
    if elapsed > 4.0:  # far below the 5 s wait limit the test sets: nothing waited for a CTA that never ran
        print(f"rank {RANK}: collectives next to compute took {elapsed:.2f} s", file=sys.stderr)
        return 1
    return 0


def case_leave_subset(comm):
    """A rank leaves between steps; the survivors see the error, form a smaller communicator and go on."""
    x = torch.ones(1 << 16, device="cuda")
    comm.allreduce(x, algo="ring", sync=True)
    if not torch.all(x == float(WS)):
        return 1
    if RANK == WS - 1:
        torch.cuda.synchronize()
        return 0
    comm.set_timeout_ms(1000)
    try:
        comm.allreduce(x, algo="ring", sync=True)
        return 1
    except ar.IbcommError as e:
        if e.code != ar.TRANSPORT_ERROR:
            return 1
    survivors = list(range(WS - 1))
    sub = ar.Communicator.from_env(tag="after", ranks=survivors)
    rc = 0
    for algo in ("ring", "rabenseifner", "direct", "oneshot", "auto"):
        n = 1 << 15 if algo == "oneshot" else 1 << 20
        y = torch.full((n,), float(RANK + 1), device="cuda")
        sub.allreduce(y, algo=algo, sync=True)
        if not torch.all(y == float(sum(r + 1 for r in survivors))):
            print(f"rank {RANK}: survivors' {algo} allreduce is wrong", file=sys.stderr)
            rc = 1
    torch.cuda.synchronize()
    sub.barrier()
    sub.close()
    return rc


def main():
    case = sys.argv[1]
    ngpu = torch.cuda.device_count()
    if ngpu < WS:
        print(f"need {WS} GPUs, have {ngpu}", file=sys.stderr)
        return 4
    torch.cuda.set_device(RANK % ngpu)
    comm = ar.Communicator.from_env()
    rc = globals()[f"case_{case}"](comm)
    torch.cuda.synchronize()
    if case not in ("leave", "leave_subset"):
        comm.barrier()
    comm.close()
    return rc


if __name__ == "__main__":
    sys.exit(main())
