"""What `auto` would pick: the library's algorithm table, queried without a GPU."""
from __future__ import annotations

import ctypes as C

from .. import _native


def choose_algorithm(nbytes: int, world_size: int, *, nvls: bool = True, mapped: bool = True,
                     max_channels: int = 0) -> tuple[str, int]:
    """(algorithm name, channels) of a device allreduce of ``nbytes`` on ``world_size`` ranks.

    ``nvls``: the box has NVSwitch multicast and the element type a switch
    reduction (fp32, fp16, bf16); ``mapped``: both buffers are mapped by the
    peers (``symmetric_empty`` or ``register``).  Honours IBCOMM_TUNING_FILE."""
    algo, ch = C.c_int(0), C.c_int(0)
    _native.check(_native.lib().ibcomm_choose_algorithm(int(nbytes), int(world_size), int(nvls), int(mapped),
                                                        int(max_channels), C.byref(algo), C.byref(ch)))
    return _native.ALGO_NAMES[algo.value], ch.value


def set_tunable(name: str, value: int) -> None:
    """Overrides one of the library's named integer knobs (``IBCOMM_NVLS_HYBRID``, ``IBCOMM_STAGED_CTAS``, ...)
    for this process; a negative value removes the override (the environment variable of the same name, then the
    built-in default, apply again).  Meant for tuning runs that compare settings without restarting."""
    _native.check(_native.lib().ibcomm_set_tunable(name.encode(), int(value)))


def get_tunable(name: str, default: int = 0) -> int:
    out = C.c_int(0)
    _native.check(_native.lib().ibcomm_get_tunable(name.encode(), int(default), C.byref(out)))
    return out.value
