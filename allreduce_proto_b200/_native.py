"""ctypes view of ``libibcomm_cuda.so`` (the C interface in ``include/ibcomm/c_api.h``).

The shared library lives in ``allreduce_proto_b200/_lib`` and is built in-tree
by :mod:`allreduce_proto_b200.build`; it is built on first import when missing.
Every C call returns one of the library's error codes, which
:func:`check` turns into :class:`IbcommError`.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "_lib"
LIB_PATH = LIB_DIR / "libibcomm_cuda.so"

INVALID_ARGUMENT = 1
TRANSPORT_ERROR = 2
IBVERBS_ERROR = 2
CUDA_ERROR = 3
NOT_SUPPORTED = 4

DTYPE_CODES = {"float32": 0, "float64": 1, "int32": 2, "int64": 3, "float16": 4, "bfloat16": 5}
ALGO_CODES = {"auto": 0, "ring": 1, "rabenseifner": 2, "nvls": 3, "oneshot": 4, "direct": 5}
ALGO_NAMES = {v: k for k, v in ALGO_CODES.items()}


class IbcommError(RuntimeError):
    """A library call failed; ``code`` is the reference's exit code (1-4)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[ibcomm error {code}] {message}")
        self.code = code
        self.message = message


class DeviceInfo(C.Structure):
    _fields_ = [("device", C.c_int), ("nvls", C.c_int), ("share_mode", C.c_int), ("last_algo", C.c_int),
                ("last_channels", C.c_int), ("pad_", C.c_int), ("arena_bytes", C.c_uint64),
                ("pool_bytes", C.c_uint64), ("work_bytes", C.c_uint64), ("calls", C.c_uint64), ("kernel_launches", C.c_uint64),
                ("switch_registrations", C.c_uint64)]


class StatusReport(C.Structure):
    _fields_ = [("code", C.c_uint32), ("kind", C.c_uint32), ("rank", C.c_int32), ("peer", C.c_int32),
                ("channel", C.c_int32), ("op_index", C.c_int32), ("expected", C.c_uint64), ("seen", C.c_uint64),
                ("seq", C.c_uint64)]


_lib = None


def _declare(lib) -> None:
    vp, sz, i, u32p, dbl = C.c_void_p, C.c_size_t, C.c_int, C.POINTER(C.c_uint32), C.c_double
    lib.ibcomm_last_error.restype = C.c_char_p
    sigs = {
        "ibcomm_has_cuda": [],
        "ibcomm_create": [i, C.POINTER(vp)],
        "ibcomm_destroy": [vp],
        "ibcomm_create_queue_pair": [vp, i, u32p],
        "ibcomm_register_queue_pair": [vp, i, u32p],
        "ibcomm_register_process": [vp, i, u32p, u32p],
        "ibcomm_register_myself": [vp, i],
        "ibcomm_set_timeout_ms": [vp, i],
        "ibcomm_set_max_channels": [vp, i],
        "ibcomm_send": [vp, i, vp, sz, i],
        "ibcomm_recv": [vp, i, vp, sz, i],
        "ibcomm_send_poll": [vp, i, C.POINTER(i)],
        "ibcomm_recv_poll": [vp, i, C.POINTER(i)],
        "ibcomm_send_wait": [vp, i],
        "ibcomm_recv_wait": [vp, i],
        "ibcomm_bcast": [vp, vp, sz, i],
        "ibcomm_barrier": [vp],
        "ibcomm_allreduce_host": [vp, i, i, vp, vp, sz],
        "ibcomm_allreduce_cuda": [vp, i, i, vp, vp, sz, dbl, i, vp, i],
        "ibcomm_choose_algorithm": [sz, i, i, i, i, C.POINTER(C.c_int), C.POINTER(C.c_int)],
        "ibcomm_reduce_scatter_host": [vp, i, vp, vp, sz],
        "ibcomm_all_gather_host": [vp, i, vp, vp, sz],
        "ibcomm_reduce_scatter_cuda": [vp, i, i, vp, vp, sz, dbl, vp, i],
        "ibcomm_all_gather_cuda": [vp, i, i, vp, vp, sz, vp, i],
        "ibcomm_check": [vp],
        "ibcomm_symmetric_alloc": [vp, sz, C.POINTER(vp)],
        "ibcomm_symmetric_free": [vp, vp],
        "ibcomm_register_buffer": [vp, vp, sz, C.POINTER(C.c_int)],
        "ibcomm_deregister_buffer": [vp, C.c_int],
        "ibcomm_get_device_info": [vp, i, C.POINTER(DeviceInfo)],
        "ibcomm_set_timer_base": [vp],
        "ibcomm_dump_trace": [vp],
        "ibcomm_staged_timeline": [vp, C.POINTER(C.c_uint64), C.c_size_t, C.POINTER(C.c_size_t)],
        "ibcomm_emu_create": [i, sz, sz, C.POINTER(vp)],
        "ibcomm_emu_destroy": [vp],
        "ibcomm_emu_allreduce": [vp, i, i, C.POINTER(vp), C.POINTER(vp), sz, dbl, i, i, vp, i],
        "ibcomm_emu_rsag": [vp, i, i, C.POINTER(vp), C.POINTER(vp), sz, dbl, i, vp, i],
        "ibcomm_emu_set_timeout_ms": [vp, i],
        "ibcomm_emu_last_channels": [vp],
        "ibcomm_emu_set_silent_rank": [vp, i],
        "ibcomm_emu_set_bad_program_rank": [vp, i],
        "ibcomm_emu_set_direct_staging": [vp, i],
        "ibcomm_emu_last_status": [vp, C.POINTER(StatusReport)],
        "ibcomm_copy_scale": [vp, vp, sz, i, i, dbl, vp],
        "ibcomm_parse_number": [C.c_char_p, C.POINTER(C.c_int64)],
        "ibcomm_get_exp_of_two": [C.c_uint64],
        "ibcomm_set_tunable": [C.c_char_p, i],
        "ibcomm_get_tunable": [C.c_char_p, i, C.POINTER(C.c_int)],
        "ibcomm_split_buffer": [sz, sz, sz, C.c_int64, C.POINTER(C.c_uint64), sz, C.POINTER(sz)],
        "ibcomm_rank_to_chunk": [sz, sz, i, C.POINTER(i), sz, C.POINTER(sz)],
        "ibcomm_describe_program": [i, i, i, sz, sz, C.c_int64, sz, C.c_char_p, sz],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_int


def lib():
    """The loaded library; builds it first when the file is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists() or os.environ.get("IBCOMM_REBUILD") == "1":
        from . import build as _build
        _build.build()
    _lib = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)
    _declare(_lib)
    return _lib


def check(code: int) -> None:
    if code != 0:
        msg = lib().ibcomm_last_error()
        raise IbcommError(code, msg.decode(errors="replace").strip() if msg else "")
