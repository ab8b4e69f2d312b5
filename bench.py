#!/usr/bin/env python
"""Headline benchmark: fp32 allreduce of one 256 MiB buffer per rank.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

One step = one out-of-place allreduce (sum, result scaled by 1/N, fused) of
67,108,864 fp32 elements per rank through the library's own kernels; the
reference's example program times exactly this operation
(examples/allreduce.cpp:21,107-118; README.md:41-51 publishes 97.5 ms on 8
nodes = 4.818 GB/s bus bandwidth).  Rank 0 prints ONE JSON line:

  value        bus bandwidth in GB/s = bytes / time * 2 (N-1) / N   (for N = 1,
               where that factor is zero, the algorithm bandwidth bytes / time of
               the fused copy+scale kernel the library runs at world size 1)
  ms_per_step  device time of one step (CUDA events around the K steps,
               barrier + synchronize on both sides, max over ranks)
  e2e          the same metric with, inside every timed step, the host->device
               copy of the 256 MiB input from pinned memory and a device->host
               read of 4 KiB of the result, through the public Communicator API
  per_algo     device-timed bus bandwidth of every algorithm the box supports
               and of NCCL (torch.distributed.all_reduce) on the same buffers
  clocks       SM clock and throttle reasons sampled with nvidia-smi during the
               timed region

`--impl reference` reports why the reference cannot run on this box.
`--sweep` runs the 4 KiB - 1 GiB message-size sweep per algorithm and writes
JSON lines to --out (default bench_out/sweep_<N>gpu.jsonl).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REFERENCE_BUSBW_GBS = 4.818  # 268435456 B / 0.0975075 s * 2 * 7 / 8, reference README.md:50
ELEMENTS = 67_108_864        # 256 MiB of fp32 (reference examples/allreduce.cpp:21)
UNAVAILABLE = ("reference is a C++/CMake library without Python packaging; its build needs libibverbs headers, "
               "an InfiniBand port with a LID, an MPI compiler wrapper and two empty submodules, none present here")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--elements", type=int, default=ELEMENTS)
    ap.add_argument("--algo", default="auto")
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--sweep-max-bytes", type=int, default=1 << 30)
    ap.add_argument("--sweep-algos", default="", help="comma-separated columns of the sweep to measure (default: all)")
    ap.add_argument("--out", default=None)
    ap.add_argument("--write-tuning", default=None, metavar="PATH",
                    help="with --sweep: write the fastest algorithm per size as an IBCOMM_TUNING_FILE table")
    ap.add_argument("--buckets", action="store_true",
                    help="time the ResNet-50 gradient-bucket allreduce (25 MiB buckets, fused 1/N, bf16-wire variant) "
                         "against NCCL on the same buckets")
    ap.add_argument("--rsag", action="store_true",
                    help="time reduce-scatter and all-gather (fp32, 1 MiB .. 1 GiB per rank in total) against NCCL")
    ap.add_argument("--no-extras", action="store_true", help="skip per-algorithm and NCCL measurements")
    ap.add_argument("--tune", default=None, metavar="SECTIONS",
                    help="sweep the kernels' knobs inside ONE process launch and write JSON lines to --out; comma-separated "
                         "sections of: hybrid, staged, mid, execmid, buffers, wire, exec, small, nccl (default with an empty string: all)")
    ap.add_argument("--p2p", action="store_true",
                    help="time device Send/Recv between ranks 0 and 1 (1 MiB .. 1 GiB) against NCCL send/recv")
    ap.add_argument("--world-sizes", action="store_true",
                    help="time ring, Rabenseifner, auto and NCCL at 64 MiB on every world size 2..N (sub-communicators of this launch)")
    ap.add_argument("--kernel-case", default=None,
                    choices=["copy", "exec_ring_emu8", "exec_rabenseifner_emu8", "oneshot_emu8", "direct_emu8",
                             "staged_emu8", "reduce_scatter_emu8", "all_gather_emu8", "noalloc_emu8"],
                    help="run one small single-GPU case of one kernel (for ncu captures) and print its time")
    return ap.parse_args()


class ClockSampler:
    """Samples `nvidia-smi` clocks and throttle reasons every 200 ms while running."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.lines: list[str] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.device_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": UNAVAILABLE}))
        return 0

    import torch
    import torch.distributed as dist

    import allreduce_proto_b200 as ar
    from allreduce_proto_b200.utils import busbw_gbs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    if args.gpus > 1 and world == 1:
        sys.stderr.write("bench.py: --gpus N > 1 must be launched with torch.distributed.run\n")
        return 2
    if not torch.cuda.is_available():
        sys.stderr.write("bench.py needs a CUDA device\n")
        return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        comm = ar.Communicator.from_torch_distributed()
    else:
        comm = ar.Communicator(1, 0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def time_steps(fn, steps: int, warmup: int) -> float:
        """ms per step: events around `steps` calls, barrier + sync on both sides, max over ranks."""
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    if args.sweep:
        return sweep(args, comm, world, rank, dev, time_steps, barrier)
    if args.rsag:
        return rsag_sweep(args, comm, world, rank, dev, time_steps)
    if args.buckets:
        return bucket_bench(args, comm, world, rank, dev, time_steps)
    if args.kernel_case:
        return kernel_case(args, comm, dev, time_steps)
    if args.tune is not None:
        return tune(args, comm, world, rank, dev, time_steps)
    if args.p2p:
        return p2p_bench(args, comm, world, rank, dev, time_steps)
    if args.world_sizes:
        return world_size_bench(args, comm, world, rank, dev, barrier, max_over_ranks)

    n = args.elements
    nbytes = n * 4
    scale = 1.0 / world
    # Buffers in the communicator's symmetric memory (zero-copy for the switch
    # path) when there are peers; plain device memory otherwise.
    if world > 1:
        sendbuf = comm.symmetric_empty(n, torch.float32)
        recvbuf = comm.symmetric_empty(n, torch.float32)
    else:
        sendbuf = torch.empty(n, dtype=torch.float32, device=dev)
        recvbuf = torch.empty(n, dtype=torch.float32, device=dev)
    sendbuf.copy_(seeded_input(n, rank, dev))

    def step():
        comm.allreduce(sendbuf, recvbuf, algo=args.algo, scale=scale)

    # Correctness of the configuration being timed (fp64 sum of the seeded inputs).
    step()
    torch.cuda.synchronize()
    comm.check()
    # A strided sample over the WHOLE buffer (every 61st element plus both ends): the two-shot kernels give
    # each rank a contiguous shard, so a prefix would only test rank 0's.
    max_err = strided_error(recvbuf, n, world, scale, dev)
    ok = max_err <= 1e-5 * world

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    # kernels of this library launched by the timed steps (the library counts them)
    launches_before = comm.device_info()["kernel_launches"]
    ms = time_steps(step, args.steps, 0)
    info = comm.device_info()
    hybrid_default = info.get("hybrid_percent", 0)
    launches = info["kernel_launches"] - launches_before
    clocks = sampler.stop() if rank == 0 else {}
    comm.check()
    value = busbw_gbs(nbytes, ms / 1e3, world)

    # End to end: pinned host input -> device, allreduce, 4 KiB of the result back.
    # The pinned buffers are placed on the GPU's own NUMA node (best effort), so that eight ranks do not
    # pull their inputs through one socket's memory.
    from allreduce_proto_b200.utils import device_numa_node
    with device_numa_node(local_rank) as numa_node:
        host_in = torch.empty(n, dtype=torch.float32, pin_memory=True)
        host_out = torch.empty(1024, dtype=torch.float32, pin_memory=True)
        host_in.zero_()
    host_in.copy_(sendbuf)

    def e2e_step():
        sendbuf.copy_(host_in, non_blocking=True)
        comm.allreduce(sendbuf, recvbuf, algo=args.algo, scale=scale)
        host_out.copy_(recvbuf[:1024], non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    e2e_ms = time_steps(e2e_step, e2e_steps, 3)
    e2e = {"value": busbw_gbs(nbytes, e2e_ms / 1e3, world), "unit": "GB/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": 4096, "steps": e2e_steps, "host_numa_node": numa_node}

    per_algo = {}
    if not args.no_extras:
        plain_in = torch.empty(n, dtype=torch.float32, device=dev)
        plain_in.copy_(sendbuf)
        plain_out = torch.empty_like(plain_in)
        k, w = max(3, args.steps // 2), 3
        if world > 1:
            candidates = [("ring", plain_in, plain_out), ("rabenseifner", plain_in, plain_out),
                          ("direct", plain_in, plain_out), ("direct_zero_copy", sendbuf, recvbuf)]
            if info["nvls"]:
                candidates += [("nvls", plain_in, plain_out)]          # staged through the pool
                candidates += [("nvls_zero_copy", sendbuf, recvbuf)]   # symmetric buffers
            for name, a, b in candidates:
                algo = name.split("_")[0]
                t = time_steps(lambda: comm.allreduce(a, b, algo=algo, scale=scale), k, w)
                per_algo[name] = {"ms": t, "busbw_gbs": busbw_gbs(nbytes, t / 1e3, world),
                                  "channels": comm.device_info()["last_channels"]}
            # Ordinary tensors registered with the communicator (CUDA IPC): no staging.
            reg_in, reg_out = plain_in.clone(), torch.empty_like(plain_in)
            rids = [comm.register(reg_in), comm.register(reg_out)]
            if min(rids) >= 0:
                t = time_steps(lambda: comm.allreduce(reg_in, reg_out, scale=scale), k, w)
                per_algo["auto_registered"] = {"ms": t, "busbw_gbs": busbw_gbs(nbytes, t / 1e3, world),
                                               "algo": comm.device_info()["last_algo"],
                                               "channels": comm.device_info()["last_channels"]}
            for rid in rids:
                comm.deregister(rid)
            del reg_in, reg_out
            t = time_steps(lambda: comm.allreduce(plain_in, plain_out, algo="ring", scale=scale, wire=torch.bfloat16), k, w)
            per_algo["ring_bf16_wire"] = {"ms": t, "busbw_gbs": busbw_gbs(nbytes, t / 1e3, world)}
            # The caller's own, unregistered tensors (the reference's contract) through `auto`.
            t = time_steps(lambda: comm.allreduce(plain_in, plain_out, scale=scale), k, w)
            per_algo["auto_plain"] = {"ms": t, "busbw_gbs": busbw_gbs(nbytes, t / 1e3, world),
                                      "algo": comm.device_info()["last_algo"], "channels": comm.device_info()["last_channels"],
                                      "max_abs_err": strided_error(plain_out, n, world, scale, dev)}
            if info["nvls"]:
                t = time_steps(lambda: comm.allreduce(plain_in, plain_out, algo="nvls", scale=scale, wire=torch.bfloat16), k, w)
                per_algo["nvls_bf16_wire"] = {"ms": t, "busbw_gbs": busbw_gbs(nbytes, t / 1e3, world)}
            nccl_buf = plain_in.clone()
            t = time_steps(lambda: dist.all_reduce(nccl_buf), k, w)
            per_algo["nccl"] = {"ms": t, "busbw_gbs": busbw_gbs(nbytes, t / 1e3, world)}
            # NCCL on memory it allocated and registered itself: zero-copy against zero-copy.
            ra, _rb, note = nccl_registered_pair(n, dev)
            if ra is not None:
                ra.copy_(plain_in)
                t = time_steps(lambda: dist.all_reduce(ra), k, w)
                per_algo["nccl_registered"] = {"ms": t, "busbw_gbs": busbw_gbs(nbytes, t / 1e3, world), "note": note}
            else:
                per_algo["nccl_registered"] = {"error": note}
        else:
            # One GPU: the same kernels with 8 emulated ranks in one cooperative
            # launch (32 MiB per rank; local memory only, so this is a kernel
            # check, not an NVLink number).
            emu = ar.EmuWorld(8)
            m = 8 << 20
            ins = [torch.rand(m, device=dev) for _ in range(8)]
            outs = [torch.empty(m, device=dev) for _ in range(8)]
            for algo in ("ring", "rabenseifner"):
                t = time_steps(lambda: emu.allreduce(ins, outs, algo=algo, scale=0.125, sync=False), k, w)
                per_algo[f"emulated8_{algo}_32MiB"] = {"ms": t, "channels": emu.last_channels}
            t = time_steps(lambda: torch.mul(sendbuf, scale, out=recvbuf), k, w)
            per_algo["torch_mul_out"] = {"ms": t, "algbw_gbs": nbytes / (t / 1e3) / 1e9}
            comm.check()

    if rank == 0:
        # Roofline of the timed kernel: one GPU = read + write of the buffer at the measured HBM copy
        # bandwidth; several GPUs = the bytes that must cross NVLink per GPU and direction (switch path
        # S (1 + 1/N), the others 2 S (N-1)/N) at the measured peer-copy bandwidth of this pool.
        roofline = None
        try:
            peaks_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
            hbm = 6650.0
            hbm_source = "fallback"
            if os.path.exists(peaks_path):
                with open(peaks_path) as f:
                    hbm = float(json.load(f).get("hbm_gbs", hbm))
                hbm_source = "measured"
            if world == 1:
                ideal_ms = 2 * nbytes / (hbm * 1e9) * 1e3
                roofline = {"bound": f"HBM copy {hbm:.0f} GB/s ({hbm_source})", "ideal_ms": ideal_ms, "fraction": ideal_ms / ms}
            else:
                # Bytes that must cross NVLink per GPU and direction: the switch path S (1 + 1/N), the hybrid
                # kernel its mix, everything else 2 S (N-1)/N.  Primary denominator: the nominal 900 GB/s per
                # direction; second column: the 770 GB/s peer copy measured on this pool.
                from allreduce_proto_b200.utils import get_tunable
                direct_share = 0.0
                if info["last_algo"] == "nvls":
                    direct_share = get_tunable("IBCOMM_NVLS_HYBRID", hybrid_default) / 100.0
                    per_dir = nbytes * ((1 - direct_share) * (1 + 1 / world) + direct_share * 2 * (world - 1) / world)
                else:
                    per_dir = 2 * nbytes * (world - 1) / world
                ideal_ms = per_dir / 900e9 * 1e3
                roofline = {"bound": "NVLink 900 GB/s per direction per GPU (nominal)", "bytes_per_direction": per_dir,
                            "direct_share_of_hybrid": direct_share, "ideal_ms": ideal_ms, "fraction": ideal_ms / ms,
                            "fraction_of_measured_770": per_dir / 770e9 * 1e3 / ms}
        except Exception:
            roofline = None
        line = {
            "metric": "allreduce_busbw_fp32_256MiB", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / REFERENCE_BUSBW_GBS, "dtype": "fp32", "data": "synthetic (uniform[-1,1), seeded by rank)",
            "config": {"model": "AllreduceCuda<float> 67,108,864 elements (256 MiB) per rank, out of place, sum * 1/N fused",
                       "global_batch": world, "seq_len": n, "parallelism": f"dp{world}",
                       "algorithm": info["last_algo"] if world > 1 else "copy+scale kernel (world size 1)",
                       "nvls": info["nvls"], "l2": "inputs (256 MiB) larger than L2 (126 MB)", "elements": n,
                       "bus_factor": "2(N-1)/N, 1 for N=1"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches), "correct": ok, "max_abs_err": max_err,
            "roofline": roofline, "per_algo": per_algo, "impl": "ours",
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        comm.close()
        dist.destroy_process_group()
    return 0 if ok else 1


def seeded_input(n: int, r: int, dev):
    """The bench's input of rank `r`: uniform[-1, 1), seeded by the rank."""
    import torch
    g = torch.Generator(device=dev)
    g.manual_seed(r)
    return torch.rand(n, dtype=torch.float32, device=dev, generator=g) * 2 - 1


def strided_error(out, n: int, world: int, scale: float, dev, stride: int = 61) -> float:
    """Largest absolute error of `out` against the fp64 sum of the ranks' seeded inputs, on every `stride`-th
    element plus the first and last 4096 (so every rank's shard and every window of a staged kernel is sampled)."""
    import torch
    idx = torch.cat([torch.arange(0, n, stride, device=dev), torch.arange(0, min(n, 4096), device=dev),
                     torch.arange(max(0, n - 4096), n, device=dev)]).unique()
    want = torch.zeros(idx.numel(), dtype=torch.float64, device=dev)
    for r in range(world):
        want += seeded_input(n, r, dev)[idx].double()
    want *= scale
    return float((out[idx].double() - want).abs().max().item())


def nccl_registered_pair(n: int, dev):
    """Two fp32 tensors of `n` elements in memory that NCCL itself allocated and registered
    (`ncclMemAlloc` through torch's MemPool, then `register_mem_pool`), so that NCCL's zero-copy
    (user-buffer registration, in-switch) paths apply to it: the counterpart of `symmetric_empty`.
    Returns (in, out, note); (None, None, reason) when this torch / NCCL cannot do it."""
    import torch
    import torch.distributed as dist
    try:
        backend = dist.group.WORLD._get_backend(dev)
        pool = torch.cuda.MemPool(backend.mem_allocator)
        with torch.cuda.use_mem_pool(pool):
            a = torch.empty(n, dtype=torch.float32, device=dev)
            b = torch.empty(n, dtype=torch.float32, device=dev)
        backend.register_mem_pool(pool)
        return a, b, "ncclMemAlloc pool registered with the communicator"
    except Exception as e:  # noqa: BLE001 - reported, not fatal
        return None, None, f"unavailable: {type(e).__name__}: {e}"


def tune(args, comm, world, rank, dev, time_steps) -> int:
    """Sweeps the knobs of the kernels inside one process launch (a launch of N ranks costs far more than a
    timed configuration).  One JSON line per configuration in --out; rank 0 prints a summary line."""
    import torch
    import torch.distributed as dist

    from allreduce_proto_b200.utils import busbw_gbs, set_tunable

    if world < 2:
        if rank == 0:
            print(json.dumps({"tune": None, "reason": "needs at least two GPUs"}))
        return 0
    sections = [x for x in args.tune.split(",") if x] or ["hybrid", "staged", "wire", "exec", "small", "nccl"]
    out_path = args.out or f"bench_out/tune_{world}gpu.jsonl"
    n = args.elements
    nbytes = n * 4
    scale = 1.0 / world
    info = comm.device_info(connect=True)
    sym_in = comm.symmetric_empty(n, torch.float32)
    sym_out = comm.symmetric_empty(n, torch.float32)
    plain_in = seeded_input(n, rank, dev)
    plain_out = torch.empty_like(plain_in)
    sym_in.copy_(plain_in)
    steps, warm = max(5, args.steps // 2), max(3, args.warmup)
    rows = []

    def run(section, name, fn, knobs=None, check=None, size=nbytes, k=steps, w=warm):
        knobs = knobs or {}
        for key, v in knobs.items():
            set_tunable(key, v)
        row = {"section": section, "name": name, "knobs": knobs, "bytes": size, "n_gpus": world}
        try:
            t = time_steps(fn, k, w)
            comm.check()
            row.update({"ms": t, "busbw_gbs": busbw_gbs(size, t / 1e3, world), "algo": comm.device_info()["last_algo"],
                        "channels": comm.device_info()["last_channels"]})
            if check is not None:
                row["max_abs_err"] = strided_error(check, size // 4, world, scale, dev)
        except Exception as e:  # noqa: BLE001 - a configuration may be unsupported
            row["error"] = str(e)
        finally:
            for key in knobs:
                set_tunable(key, -1)
        rows.append(row)
        return row

    def allreduce(a, b, algo, wire=None):
        return lambda: comm.allreduce(a, b, algo=algo, scale=scale, wire=wire)

    if "nccl" in sections:
        buf = plain_in.clone()
        run("nccl", "nccl_plain", lambda: dist.all_reduce(buf))
        ra, rb, note = nccl_registered_pair(n, dev)
        if ra is not None:
            ra.copy_(plain_in)
            r = run("nccl", "nccl_registered", lambda: dist.all_reduce(ra))
            r["note"] = note
        else:
            rows.append({"section": "nccl", "name": "nccl_registered", "error": note})
        del buf
    if "hybrid" in sections and info["nvls"]:
        run("hybrid", "nvls_zero_copy", allreduce(sym_in, sym_out, "nvls"), {"IBCOMM_NVLS_HYBRID": 0}, check=sym_out)
        run("hybrid", "direct_zero_copy", allreduce(sym_in, sym_out, "direct"), check=sym_out)
        splits = ((32, 96), (48, 96), (64, 84), (48, 64), (24, 120)) if world > 2 else ((48, 96), (32, 112))
        for pct in (10, 15, 20, 25, 30, 35, 40, 50):
            for a, b in splits:
                run("hybrid", f"hybrid_{pct}_{a}_{b}", allreduce(sym_in, sym_out, "nvls"),
                    {"IBCOMM_NVLS_HYBRID": pct, "IBCOMM_NVLS_HYBRID_SWITCH_CTAS": a, "IBCOMM_NVLS_HYBRID_DIRECT_CTAS": b},
                    check=sym_out if (a, b) == splits[0] else None)
        for ch in (32, 64, 96, 128):
            run("hybrid", f"direct_zero_copy_ch{ch}", allreduce(sym_in, sym_out, "direct"), {"IBCOMM_TWOSHOT_CHANNELS": ch})
    if "staged" in sections:
        algos = ["direct"] + (["nvls"] if info["nvls"] else [])
        for algo in algos:
            run("staged", f"{algo}_sequential", allreduce(plain_in, plain_out, algo), {"IBCOMM_STAGED": 0}, check=plain_out)
            for ctas in (64, 96, 128, 148):
                for tma in (1, 0):
                    run("staged", f"{algo}_pipelined_ctas{ctas}_tma{tma}", allreduce(plain_in, plain_out, algo),
                        {"IBCOMM_STAGED_CTAS": ctas, "IBCOMM_STAGED_TMA": tma}, check=plain_out if ctas == 128 else None)
            for kib in (4096, 8192, 16384):
                run("staged", f"{algo}_pipelined_window{kib}KiB", allreduce(plain_in, plain_out, algo),
                    {"IBCOMM_STAGED_WINDOW_KIB": kib})
        for size in (1 << 20, 4 << 20, 16 << 20, 64 << 20):
            m = size // 4
            for algo in algos + ["auto", "ring", "rabenseifner"]:
                run("staged", f"{algo}_plain_{size >> 20}MiB", allreduce(plain_in[:m], plain_out[:m], algo), size=size, k=30, w=5)
            nb = plain_in[:m].clone()
            run("staged", f"nccl_{size >> 20}MiB", lambda: dist.all_reduce(nb), size=size, k=30, w=5)
    if "mid" in sections:
        # Medium messages in ordinary buffers: window size of the pipelined staged kernel against the
        # zero-copy kernels (the floor), the op programs and NCCL.
        algos = ["direct"] + (["nvls"] if info["nvls"] else [])
        for size in (32 << 20, 64 << 20, 128 << 20):
            m = size // 4
            if m > n:
                continue
            for algo in algos:
                run("mid", f"{algo}_zero_copy_{size >> 20}MiB", allreduce(sym_in[:m], sym_out[:m], algo), size=size, k=30, w=5)
                for kib in (0, 2048, 4096, 8192):
                    for ctas in (64, 128):
                        run("mid", f"{algo}_window{kib}KiB_ctas{ctas}_{size >> 20}MiB", allreduce(plain_in[:m], plain_out[:m], algo),
                            {"IBCOMM_STAGED_WINDOW_KIB": kib, "IBCOMM_STAGED_CTAS": ctas}, size=size, k=30, w=5,
                            check=plain_out[:m] if kib == 4096 and ctas == 64 else None)
            for algo in ("auto", "ring", "rabenseifner"):
                run("mid", f"{algo}_plain_{size >> 20}MiB", allreduce(plain_in[:m], plain_out[:m], algo), size=size, k=30, w=5)
            nb = plain_in[:m].clone()
            run("mid", f"nccl_{size >> 20}MiB", lambda: dist.all_reduce(nb), size=size, k=30, w=5)
    if "pipe" in sections:
        # Shapes of the pipelined staged kernel on ordinary buffers: roles in every block or in blocks of
        # their own, windows of each kind, groups per role, poster warps, bulk copies against register copies.
        algo = "nvls" if info["nvls"] and world > 2 else "direct"
        shapes = [("roles_in_every_block_bufs3", {"IBCOMM_STAGED_SPLIT": 0, "IBCOMM_STAGED_BUFFERS": 3})]
        for bufs, lg, rg in ((3, 1, 2), (4, 2, 2), (6, 1, 2), (6, 2, 2), (6, 3, 2)):
            for posters in (0, 1):
                for tma in (1, 0):
                    shapes.append((f"split_bufs{bufs}_groups{lg}_{rg}_{lg}_posters{posters}_tma{tma}",
                                   {"IBCOMM_STAGED_SPLIT": 1, "IBCOMM_STAGED_BUFFERS": bufs, "IBCOMM_STAGED_LOAD_GROUPS": lg,
                                    "IBCOMM_STAGED_REDUCE_GROUPS": rg, "IBCOMM_STAGED_STORE_GROUPS": lg,
                                    "IBCOMM_STAGED_POSTERS": posters, "IBCOMM_STAGED_TMA": tma}))
        for size in (64 << 20, 256 << 20):
            m = size // 4
            if m > n:
                continue
            for name, knobs in shapes:
                run("pipe", f"{algo}_{name}_{size >> 20}MiB", allreduce(plain_in[:m], plain_out[:m], algo), knobs, size=size, k=20, w=4,
                    check=plain_out[:m] if name.endswith("posters1_tma1") and name.startswith("split_bufs6_groups3") else None)
            run("pipe", f"{algo}_zero_copy_{size >> 20}MiB", allreduce(sym_in[:m], sym_out[:m], algo), size=size, k=20, w=4)
            nb = plain_in[:m].clone()
            run("pipe", f"nccl_{size >> 20}MiB", lambda: dist.all_reduce(nb), size=size, k=20, w=4)
    if "execmid" in sections:
        # The op programs at medium sizes: CTAs x threads per CTA (per-op overhead against parallelism).
        for size in (16 << 20, 64 << 20):
            m = size // 4
            for algo in ("ring", "rabenseifner"):
                for threads in (512, 256):
                    for ch in (32, 64, 96, 128, 148, 256):
                        run("execmid", f"{algo}_t{threads}_ch{ch}_{size >> 20}MiB", allreduce(plain_in[:m], plain_out[:m], algo),
                            {"IBCOMM_EXEC_THREADS": threads, "IBCOMM_EXEC_CHANNELS": ch}, size=size, k=30, w=5)
    if "buffers" in sections:
        # The pipelined staged kernel: window buffers of each kind x CTAs (ordinary buffers, full size).
        for algo in (["nvls"] if info["nvls"] else ["direct"]):
            for bufs in (3, 4, 6):
                for ctas in (48, 64, 96, 128):
                    run("buffers", f"{algo}_pipelined_bufs{bufs}_ctas{ctas}", allreduce(plain_in, plain_out, algo),
                        {"IBCOMM_STAGED_BUFFERS": bufs, "IBCOMM_STAGED_CTAS": ctas}, check=plain_out if ctas == 64 else None)
    if "wire" in sections:
        for algo in ["ring", "rabenseifner", "direct"] + (["nvls"] if info["nvls"] else []):
            for wire in (torch.bfloat16, torch.float16):
                r = run("wire", f"{algo}_{str(wire).split('.')[-1]}_wire", allreduce(plain_in, plain_out, algo, wire=wire))
                if "error" not in r:
                    r["max_abs_err"] = strided_error(plain_out, n, world, scale, dev)
        if info["nvls"]:
            for ctas in (64, 96, 148):
                run("wire", f"nvls_bfloat16_wire_ctas{ctas}", allreduce(plain_in, plain_out, "nvls", wire=torch.bfloat16),
                    {"IBCOMM_STAGED_CTAS": ctas})
    if "exec" in sections:
        for algo in ("ring", "rabenseifner"):
            for threads in (512, 256):
                for ch in (64, 128, 148, 256):
                    run("exec", f"{algo}_t{threads}_ch{ch}", allreduce(plain_in, plain_out, algo),
                        {"IBCOMM_EXEC_THREADS": threads, "IBCOMM_EXEC_CHANNELS": ch}, check=plain_out if ch == 256 else None)
        for pos in (2, 8):
            run("exec", f"ring_positions{pos}", allreduce(plain_in, plain_out, "ring"), {"IBCOMM_RING_POSITIONS": pos}, check=plain_out)
        for pieces in (2, 4, 16):
            run("exec", f"rabenseifner_pieces{pieces}", allreduce(plain_in, plain_out, "rabenseifner"),
                {"IBCOMM_RABEN_PIECES": pieces}, check=plain_out)
    if "small" in sections:
        for size in (4 << 10, 64 << 10, 1 << 20):
            m = size // 4
            for algo in ("ring", "rabenseifner", "oneshot", "auto"):
                if algo == "oneshot" and size > (512 << 10):
                    continue
                run("small", f"{algo}_{size >> 10}KiB", allreduce(plain_in[:m], plain_out[:m], algo), size=size, k=200, w=20)
            nb = plain_in[:m].clone()
            run("small", f"nccl_{size >> 10}KiB", lambda: dist.all_reduce(nb), size=size, k=200, w=20)
    if rank == 0:
        os.makedirs(os.path.dirname(out_path) or ".", exist_ok=True)
        with open(out_path, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
        best = {}
        for r in rows:
            if "ms" in r and r["bytes"] == nbytes and (r["section"] not in best or r["ms"] < best[r["section"]]["ms"]):
                best[r["section"]] = r
        print(json.dumps({"tune": out_path, "rows": len(rows), "n_gpus": world,
                          "best": {k: {"name": v["name"], "ms": v["ms"], "busbw_gbs": v["busbw_gbs"]} for k, v in best.items()}}))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


def p2p_bench(args, comm, world, rank, dev, time_steps) -> int:
    """Device Send/Recv between ranks 0 and 1: one direction, and both directions at once, 1 MiB .. 1 GiB,
    against NCCL's send/recv on the same tensors.  Device time (CUDA events on the default stream, which the
    library's blocking send and receive streams synchronise with), max over ranks."""
    import torch
    import torch.distributed as dist

    if world < 2:
        if rank == 0:
            print(json.dumps({"p2p": None, "reason": "needs at least two GPUs"}))
        return 0
    out_path = args.out or f"bench_out/p2p_{world}gpu.jsonl"
    nmax = min(args.sweep_max_bytes, 1 << 30)
    src = torch.empty(nmax, dtype=torch.uint8, device=dev)
    dst = torch.empty(nmax, dtype=torch.uint8, device=dev)
    src.copy_(torch.arange(nmax, device=dev, dtype=torch.int64).remainder(251).to(torch.uint8) + rank)
    comm.device_info(connect=True)
    rows = []
    size = 1 << 20
    while size <= nmax:
        a, b = src[:size], dst[:size]
        steps, warm = (50, 5) if size <= (64 << 20) else (10, 3)

        def one_way():
            if rank == 0:
                comm.send(1, a, blocking=False)
                comm.send_wait(1)
            elif rank == 1:
                comm.recv(0, b, blocking=True)

        def both_ways():
            if rank < 2:
                comm.send(1 - rank, a, blocking=False)
                comm.recv(1 - rank, b, blocking=True)
                comm.send_wait(1 - rank)

        def nccl_one_way():
            if rank == 0:
                dist.send(a, 1)
            elif rank == 1:
                dist.recv(b, 0)

        for name, fn, dirs in (("ours_one_way", one_way, 1), ("ours_both_ways", both_ways, 1), ("nccl_one_way", nccl_one_way, 1)):
            t = time_steps(fn, steps, warm)
            comm.check()
            rows.append({"bytes": size, "name": name, "us": t * 1e3, "gbs_per_direction": size * dirs / (t / 1e3) / 1e9})
        if rank == 1:
            want = (torch.arange(size, device=dev, dtype=torch.int64).remainder(251).to(torch.uint8))
            if not torch.equal(b, want):
                rows.append({"bytes": size, "name": "payload_mismatch"})
        size *= 4
    if rank == 0:
        os.makedirs(os.path.dirname(out_path) or ".", exist_ok=True)
        with open(out_path, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
        print(json.dumps({"p2p": out_path, "rows": len(rows),
                          "at_largest": {r["name"]: round(r["gbs_per_direction"], 1) for r in rows if r["bytes"] == size // 4 and "us" in r}}))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


def world_size_bench(args, comm, world, rank, dev, barrier, max_over_ranks) -> int:
    """Ring, Rabenseifner, auto and NCCL at 64 MiB of fp32 (normal(0, 1) values seeded by rank) on every world
    size 2..N of this launch, the non-powers of two included: a communicator over the first w ranks each
    (the other ranks wait at a barrier of the whole job).  Checked against the fp64 sum."""
    import torch
    import torch.distributed as dist

    import allreduce_proto_b200 as ar
    from allreduce_proto_b200.utils import busbw_gbs

    out_path = args.out or f"bench_out/world_sizes_{world}gpu.jsonl"
    n = (64 << 20) // 4
    g = torch.Generator(device=dev)
    g.manual_seed(rank)
    x = torch.randn(n, device=dev, generator=g)
    y = torch.empty_like(x)
    rows = []
    for w in range(2, world + 1):
        members = list(range(w))
        group = dist.new_group(members)  # every rank of the job takes part in creating it
        if rank < w:
            sub = comm if w == world else ar.Communicator.from_torch_distributed(tag=f"ws{w}", ranks=members)
            want = torch.zeros(n, dtype=torch.float64, device=dev)
            for r in range(w):
                gr = torch.Generator(device=dev)
                gr.manual_seed(r)
                want += torch.randn(n, device=dev, generator=gr).double()
            for algo in ("ring", "rabenseifner", "auto", "nccl"):
                def step():
                    if algo == "nccl":
                        dist.all_reduce(y, group=group)  # in place, on the previous result: timing only
                    else:
                        sub.allreduce(x, y, algo=algo)
                for _ in range(5):
                    step()
                torch.cuda.synchronize()
                dist.barrier(group=group)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                steps = 20
                e0.record()
                for _ in range(steps):
                    step()
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                ms = float(t.item())
                if algo != "nccl":
                    sub.check()
                err = float((y.double() - want).abs().max().item()) if algo != "nccl" else None
                rows.append({"world_size": w, "algo": algo, "bytes": n * 4, "ms": ms, "busbw_gbs": busbw_gbs(n * 4, ms / 1e3, w),
                             "max_abs_err": err, "chosen": sub.device_info()["last_algo"] if algo != "nccl" else "nccl"})
            if sub is not comm:
                sub.barrier()
                sub.close()
        barrier()
    if rank == 0:
        os.makedirs(os.path.dirname(out_path) or ".", exist_ok=True)
        with open(out_path, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
        print(json.dumps({"world_sizes": out_path, "rows": len(rows)}))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


def kernel_case(args, comm, dev, time_steps) -> int:
    """One kernel, one GPU, small inputs (still larger than L2): the workload of the ncu captures in profiles/."""
    import torch

    import allreduce_proto_b200 as ar

    case = args.kernel_case
    if case == "copy":
        n = 64 << 20  # 256 MiB in, 256 MiB out
        x = torch.rand(n, device=dev)
        y = torch.empty_like(x)
        ms = time_steps(lambda: comm.allreduce(x, y, scale=0.5), args.steps, args.warmup)
        moved = 2 * n * 4
    elif case == "noalloc_emu8":
        # The allocation-free entry point (include/ibcomm/no_alloc.h): 8 emulated ranks x 32 KiB, its limit.
        import ctypes as C

        from allreduce_proto_b200 import _native
        fn = _native.lib().ibcomm_emu_oneshot_allreduce_f32_noalloc
        fn.restype = C.c_int
        fn.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_float, C.c_void_p, C.c_char_p, C.c_size_t]
        ins = [torch.rand(8192, device=dev) for _ in range(8)]
        outs = [torch.empty(8192, device=dev) for _ in range(8)]
        pin = (C.c_void_p * 8)(*[t.data_ptr() for t in ins])
        pout = (C.c_void_p * 8)(*[t.data_ptr() for t in outs])
        err = C.create_string_buffer(256)

        def step():
            if fn(pin, pout, 8, 8192, 0.125, C.c_void_p(torch.cuda.current_stream().cuda_stream), err, len(err)) != 0:
                raise RuntimeError(err.value.decode())
        ms = time_steps(step, args.steps, args.warmup)
        want = torch.stack(ins).sum(0) * 0.125
        assert torch.allclose(outs[3], want, rtol=1e-5, atol=1e-6)
        moved = None
    elif case in ("reduce_scatter_emu8", "all_gather_emu8"):
        emu = ar.EmuWorld(8)
        m = 1 << 20  # elements per block: 32 MiB per rank in the full buffers
        full = [torch.rand(8 * m, device=dev) for _ in range(8)]
        shard = [torch.rand(m, device=dev) for _ in range(8)]
        if case == "reduce_scatter_emu8":
            ms = time_steps(lambda: emu.reduce_scatter(full, shard, scale=0.125), args.steps, args.warmup)
        else:
            ms = time_steps(lambda: emu.all_gather(shard, full), args.steps, args.warmup)
        moved = None
    else:
        emu = ar.EmuWorld(8)
        algo = {"exec_ring_emu8": "ring", "exec_rabenseifner_emu8": "rabenseifner", "oneshot_emu8": "oneshot",
                "direct_emu8": "direct", "staged_emu8": "direct"}[case]
        if case == "staged_emu8":
            emu.set_direct_staging(2)  # the pipelined staged kernel: copy in, peer reduce and copy out overlap
        m = (16 << 10) if algo == "oneshot" else (8 << 20)  # elements per rank: 64 KiB or 32 MiB
        ins = [torch.rand(m, device=dev) for _ in range(8)]
        outs = [torch.empty(m, device=dev) for _ in range(8)]
        ms = time_steps(lambda: emu.allreduce(ins, outs, algo=algo, scale=0.125, sync=False), args.steps, args.warmup)
        moved = None
    print(json.dumps({"kernel_case": case, "ms": ms, "steps": args.steps,
                      "gbs_read_plus_write": (moved / (ms / 1e3) / 1e9) if moved else None}))
    return 0


def bucket_bench(args, comm, world, rank, dev, time_steps) -> int:
    """The data-parallel gradient workload: ResNet-50's 161 gradient tensors (25.6 M fp32 values, ~N(0, 1e-3))
    in 25 MiB buckets, summed over the ranks with the 1/N scale fused; fp32 on the wire, bf16 on the wire, the
    sharded pair (reduce-scatter + all-gather), and NCCL (`all_reduce` of every bucket followed by the scale)."""
    import torch
    import torch.distributed as dist

    import allreduce_proto_b200 as ar
    from allreduce_proto_b200.models import resnet50_param_shapes, synthetic_grads

    shapes = [s for _, s in resnet50_param_shapes()]
    grads = synthetic_grads(dev, seed=rank)
    steps, warm = max(5, args.steps), max(3, args.warmup)
    out = {"workload": "resnet50_gradient_buckets", "n_gpus": world, "tensors": len(shapes), "bucket_bytes": 25 << 20}
    sym = ar.GradientBuckets(shapes, comm=comm, bucket_bytes=25 << 20, shardable=True)
    sym.load(grads)
    out["buckets"] = sym.num_buckets
    out["bytes"] = sym.nbytes
    t = time_steps(lambda: sym.allreduce(average=True), steps, warm)
    out["allreduce_fp32_ms"] = t
    if world > 1:
        t = time_steps(lambda: sym.allreduce(average=True, wire=torch.bfloat16), steps, warm)
        out["allreduce_bf16_wire_ms"] = t
        t = time_steps(lambda: (sym.reduce_scatter(average=True), sym.all_gather()), steps, warm)
        out["reduce_scatter_plus_all_gather_ms"] = t
        plain = ar.GradientBuckets(shapes, comm=comm, bucket_bytes=25 << 20, symmetric=False)
        plain.load(grads)
        t = time_steps(lambda: plain.allreduce(average=True), steps, warm)
        out["allreduce_fp32_ordinary_tensors_ms"] = t
        rids = [comm.register(b) for b in plain.flat]
        if min(rids) >= 0:
            t = time_steps(lambda: plain.allreduce(average=True), steps, warm)
            out["allreduce_fp32_registered_tensors_ms"] = t
        for rid in rids:
            if rid >= 0:
                comm.deregister(rid)

        def nccl_step():
            for b in plain.flat:
                dist.all_reduce(b)
            torch._foreach_mul_(plain.flat, 1.0 / world)
        t = time_steps(nccl_step, steps, warm)
        out["nccl_all_reduce_plus_scale_ms"] = t
    comm.check()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        comm.close()
        dist.destroy_process_group()
    return 0


def rsag_sweep(args, comm, world, rank, dev, time_steps) -> int:
    """Reduce-scatter and all-gather, fp32: symmetric, registered and ordinary tensors, and NCCL's
    reduce_scatter_tensor / all_gather_into_tensor on the same box.  `bytes` is the size of the full
    (world_size blocks) buffer; bus bandwidth = bytes / time x (N-1)/N."""
    import torch
    import torch.distributed as dist

    if world < 2:
        if rank == 0:
            print(json.dumps({"rsag": None, "reason": "needs at least two GPUs"}))
        return 0
    out_path = args.out or f"bench_out/rsag_{world}gpu.jsonl"
    max_bytes = min(args.sweep_max_bytes, 1 << 30)
    nmax = max_bytes // 4
    full = {"symmetric": comm.symmetric_empty(nmax, torch.float32), "plain": torch.empty(nmax, device=dev),
            "registered": torch.empty(nmax, device=dev)}
    rid = comm.register(full["registered"])
    if rid < 0:
        del full["registered"]
    g = torch.Generator(device=dev)
    g.manual_seed(rank)
    full["plain"].copy_(torch.rand(nmax, device=dev, generator=g) * 2 - 1)
    for k in full:
        if k != "plain":
            full[k].copy_(full["plain"])
    shard = torch.empty(nmax // world, device=dev)
    nccl_full = full["plain"].clone()
    burn = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
    t_end = time.time() + 1.0
    while time.time() < t_end:
        for _ in range(20):
            burn @ burn
        torch.cuda.synchronize()
    del burn
    rows = []
    size = 1 << 20
    while size <= max_bytes:
        m = size // 4 // world
        n = m * world
        steps, warm = (100, 10) if size <= (16 << 20) else (20, 5)
        factor = (world - 1) / world
        for kind, buf in full.items():
            t = time_steps(lambda: comm.reduce_scatter(buf[:n], shard[:m], scale=1.0 / world), steps, warm)
            comm.check()
            rows.append({"bytes": n * 4, "op": "reduce_scatter", "buffers": kind, "us": t * 1e3,
                         "busbw_gbs": n * 4 * factor / (t / 1e3) / 1e9, "algo": comm.device_info()["last_algo"]})
            t = time_steps(lambda: comm.all_gather(shard[:m], buf[:n]), steps, warm)
            comm.check()
            rows.append({"bytes": n * 4, "op": "all_gather", "buffers": kind, "us": t * 1e3,
                         "busbw_gbs": n * 4 * factor / (t / 1e3) / 1e9, "algo": comm.device_info()["last_algo"]})
        t = time_steps(lambda: dist.reduce_scatter_tensor(shard[:m], nccl_full[:n]), steps, warm)
        rows.append({"bytes": n * 4, "op": "reduce_scatter", "buffers": "nccl", "us": t * 1e3,
                     "busbw_gbs": n * 4 * factor / (t / 1e3) / 1e9})
        t = time_steps(lambda: dist.all_gather_into_tensor(nccl_full[:n], shard[:m]), steps, warm)
        rows.append({"bytes": n * 4, "op": "all_gather", "buffers": "nccl", "us": t * 1e3,
                     "busbw_gbs": n * 4 * factor / (t / 1e3) / 1e9})
        size *= 4
    if rank == 0:
        os.makedirs(os.path.dirname(out_path) or ".", exist_ok=True)
        with open(out_path, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
        print(json.dumps({"rsag": out_path, "rows": len(rows), "n_gpus": world}))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    return 0


def sweep(args, comm, world, rank, dev, time_steps, barrier) -> int:
    """Message-size sweep 4 KiB .. 1 GiB (powers of two), fp32, every algorithm and NCCL."""
    import torch
    import torch.distributed as dist

    from allreduce_proto_b200.utils import busbw_gbs

    out_path = args.out or f"bench_out/sweep_{world}gpu.jsonl"
    info = comm.device_info(connect=world > 1)
    rows = []
    max_bytes = args.sweep_max_bytes
    nmax = max_bytes // 4
    if world > 1:
        sym_in = comm.symmetric_empty(nmax, torch.float32)
        sym_out = comm.symmetric_empty(nmax, torch.float32)
    else:
        sym_in = torch.empty(nmax, dtype=torch.float32, device=dev)
        sym_out = torch.empty(nmax, dtype=torch.float32, device=dev)
    plain_in = torch.empty(nmax, dtype=torch.float32, device=dev)
    plain_out = torch.empty(nmax, dtype=torch.float32, device=dev)
    g = torch.Generator(device=dev)
    g.manual_seed(rank)
    plain_in.copy_(torch.rand(nmax, dtype=torch.float32, device=dev, generator=g) * 2 - 1)
    sym_in.copy_(plain_in)
    nccl_buf = torch.empty(nmax, dtype=torch.float32, device=dev)
    nccl_reg = None
    if world > 1:
        nccl_reg, _unused, nccl_reg_note = nccl_registered_pair(nmax, dev)
        del _unused
    registered = False
    if world > 1:
        reg_in, reg_out = plain_in.clone(), torch.empty_like(plain_in)
        registered = min(comm.register(reg_in), comm.register(reg_out)) >= 0
    # Bring the clocks up before the smallest (latency-bound) sizes are timed.
    burn = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
    t_end = time.time() + 1.0
    while time.time() < t_end:
        for _ in range(20):
            burn @ burn
        torch.cuda.synchronize()
    del burn
    size = 4096
    while size <= max_bytes:
        n = size // 4
        steps = 200 if size <= (1 << 20) else (50 if size <= (64 << 20) else 10)
        warm = 20 if size <= (1 << 20) else 5
        algos = []
        if world > 1:
            if size <= (512 << 10):
                algos.append(("oneshot", plain_in, plain_out))
            algos += [("ring", plain_in, plain_out), ("rabenseifner", plain_in, plain_out),
                      ("direct", plain_in, plain_out), ("direct_zero_copy", sym_in, sym_out)]
            if info["nvls"]:
                algos += [("nvls", plain_in, plain_out), ("nvls_zero_copy", sym_in, sym_out)]
            algos.append(("auto_plain", plain_in, plain_out))
            if registered:
                algos.append(("auto_registered", reg_in, reg_out))
            algos.append(("auto", sym_in, sym_out))
        else:
            algos.append(("auto", plain_in, plain_out))
        only = [s for s in args.sweep_algos.split(",") if s]
        for name, a, b in algos:
            if only and name not in only:
                continue
            algo = name.split("_")[0]
            try:
                t = time_steps(lambda: comm.allreduce(a[:n], b[:n], algo=algo, scale=1.0 / world), steps, warm)
                comm.check()
            except Exception as e:  # an algorithm may be unavailable for a size
                rows.append({"bytes": size, "algo": name, "error": str(e)})
                continue
            rows.append({"bytes": size, "algo": name, "us": t * 1e3, "busbw_gbs": busbw_gbs(size, t / 1e3, world),
                         "algbw_gbs": size / (t / 1e3) / 1e9, "chosen": comm.device_info()["last_algo"],
                         "channels": comm.device_info()["last_channels"], "n_gpus": world})
        if world > 1:
            t = time_steps(lambda: dist.all_reduce(nccl_buf[:n]), steps, warm)
            rows.append({"bytes": size, "algo": "nccl", "us": t * 1e3, "busbw_gbs": busbw_gbs(size, t / 1e3, world),
                         "algbw_gbs": size / (t / 1e3) / 1e9, "n_gpus": world})
            if nccl_reg is not None:
                t = time_steps(lambda: dist.all_reduce(nccl_reg[:n]), steps, warm)
                rows.append({"bytes": size, "algo": "nccl_registered", "us": t * 1e3, "busbw_gbs": busbw_gbs(size, t / 1e3, world),
                             "algbw_gbs": size / (t / 1e3) / 1e9, "n_gpus": world})
        size *= 2
    if rank == 0:
        os.makedirs(os.path.dirname(out_path) or ".", exist_ok=True)
        with open(out_path, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
        print(json.dumps({"sweep": out_path, "rows": len(rows), "n_gpus": world, "nvls": info["nvls"]}))
        if args.write_tuning and world > 1:
            write_tuning(args.write_tuning, rows, world)
    if world > 1:
        dist.barrier()
        comm.close()
        dist.destroy_process_group()
    return 0


def write_tuning(path: str, rows: list, world: int) -> None:
    """IBCOMM_TUNING_FILE table ("world_size max_bytes algorithm channels", first match wins) from a sweep:
    per size the fastest algorithm measured on symmetric buffers (plain-buffer columns where there is no
    symmetric variant); consecutive sizes with the same choice are merged."""
    best = []
    for size in sorted({r["bytes"] for r in rows}):
        cands = [r for r in rows if r["bytes"] == size and "us" in r and r["algo"] in
                 ("oneshot", "ring", "rabenseifner", "direct_zero_copy", "nvls_zero_copy")]
        if cands:
            w = min(cands, key=lambda r: r["us"])
            best.append((size, w["algo"].split("_")[0], int(w.get("channels") or 0)))
    lines = ["# world_size max_bytes algorithm channels   (written by bench.py --sweep --write-tuning)"]
    for i, (size, algo, ch) in enumerate(best):
        last = i + 1 == len(best)
        if not last and best[i + 1][1] == algo:
            continue
        lines.append(f"{world} {0 if last else size} {algo} 0")
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    sys.exit(main())
