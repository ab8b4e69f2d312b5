"""Size strings (``"128M"``, ``"31kb"``) as the tester understands them."""
from __future__ import annotations

import ctypes as C

from .. import _native


def parse_number(text: str) -> int:
    """``[+-]digits[k|m|g][b]`` with binary multipliers; raises ``ValueError`` otherwise.

    Same grammar as the reference's ``util::parse_number`` (ibcomm/util.h:81-149).
    """
    out = C.c_int64(0)
    if _native.lib().ibcomm_parse_number(text.encode(), C.byref(out)) != 0:
        raise ValueError(_native.lib().ibcomm_last_error().decode())
    return out.value


def get_exp_of_two(n: int) -> int:
    """p when n == 2**p, else 0 (so 1 and 0 give 0): reference ibcomm/util.h:156-175."""
    return _native.lib().ibcomm_get_exp_of_two(n)


def format_bytes(n: int) -> str:
    for unit, shift in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if n >= (1 << shift) and n % (1 << shift) == 0:
            return f"{n >> shift} {unit}"
    return f"{n} B"
