"""NUMA placement of host buffers that feed a GPU.

On a two-socket box with eight GPUs, pinned host memory that lives on the
other socket than the GPU crosses the socket interconnect on every
host-to-device copy, and when every rank's buffers sit on ONE socket the
copies of all GPUs share that socket's memory bandwidth.  `device_numa_node`
is a context manager that, while host buffers are being allocated, prefers
the memory of the GPU's own NUMA node (``set_mempolicy(MPOL_PREFERRED)``) and
runs the allocating thread on that node's cores; both are restored on exit.
Everything is best effort: without the sysfs entries, on a single-node
machine, or when the calls are not permitted, it does nothing and yields
``None``.  The reference leaves placement to the MPI launcher's binding
options."""
from __future__ import annotations

import contextlib
import ctypes
import os
from typing import Iterator, Optional

_SYS_SET_MEMPOLICY = {"x86_64": 238, "aarch64": 237}
_MPOL_DEFAULT, _MPOL_PREFERRED = 0, 1


def _parse_cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            lo, hi = part.split("-")
            cpus.update(range(int(lo), int(hi) + 1))
        else:
            cpus.add(int(part))
    return cpus


def numa_node_of_device(device: int) -> Optional[int]:
    """NUMA node of CUDA device ``device`` from sysfs, or ``None`` when unknown."""
    try:
        import torch
        p = torch.cuda.get_device_properties(device)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        return node if node >= 0 else None
    except Exception:
        return None


def _set_mempolicy(mode: int, node: Optional[int]) -> bool:
    nr = _SYS_SET_MEMPOLICY.get(os.uname().machine)
    if nr is None:
        return False
    try:
        libc = ctypes.CDLL(None, use_errno=True)
        if node is None:
            return libc.syscall(ctypes.c_long(nr), ctypes.c_int(mode), ctypes.c_void_p(0), ctypes.c_ulong(0)) == 0
        mask = (ctypes.c_ulong * 16)()
        bits = 8 * ctypes.sizeof(ctypes.c_ulong)
        if node >= 16 * bits:
            return False
        mask[node // bits] = 1 << (node % bits)
        return libc.syscall(ctypes.c_long(nr), ctypes.c_int(mode), mask, ctypes.c_ulong(16 * bits)) == 0
    except Exception:
        return False


@contextlib.contextmanager
def device_numa_node(device: int) -> Iterator[Optional[int]]:
    """Prefer the NUMA node of CUDA device ``device`` for allocations made inside the block.

    Yields the node, or ``None`` when nothing was changed."""
    node = numa_node_of_device(device)
    if node is None:
        yield None
        return
    policy_set = _set_mempolicy(_MPOL_PREFERRED, node)
    old_affinity = None
    try:
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            local = _parse_cpulist(f.read())
        allowed = os.sched_getaffinity(0)
        if local & allowed and (local & allowed) != allowed:
            old_affinity = allowed
            os.sched_setaffinity(0, local & allowed)
    except Exception:
        old_affinity = None
    try:
        yield node if (policy_set or old_affinity is not None) else None
    finally:
        if old_affinity is not None:
            try:
                os.sched_setaffinity(0, old_affinity)
            except Exception:
                pass
        if policy_set:
            _set_mempolicy(_MPOL_DEFAULT, None)
