"""The allocation-free allreduce entry point (include/ibcomm/no_alloc.h), called
through its exported C symbol and compared with the regular one-shot path
(EmuWorld) on two calls in a row.  Both add the ranks' copies in rank order in
fp32, so the results must agree to the last bit; the tolerance used is the one
of the other fp32 tests.  The file name makes pytest collect it last."""
import ctypes as C

import pytest
import torch

import allreduce_proto_b200 as ar
from allreduce_proto_b200 import _native

pytestmark = pytest.mark.gpu


def call_no_alloc(sendbufs, recvbufs, scale):
    lib = _native.lib()
    fn = lib.ibcomm_emu_oneshot_allreduce_f32_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_float, C.c_void_p, C.c_char_p, C.c_size_t]
    ws = len(sendbufs)
    ins = (C.c_void_p * ws)(*[t.data_ptr() for t in sendbufs])
    outs = (C.c_void_p * ws)(*[t.data_ptr() for t in recvbufs])
    err = C.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    code = fn(ins, outs, ws, sendbufs[0].numel(), scale, C.c_void_p(stream), err, len(err))
    return code, err.value.decode()


def test_no_alloc_entry_matches_regular_path_twice():
    ws = 4
    world = ar.EmuWorld(ws, 1 << 20, 1 << 20)
    g = torch.Generator(device="cuda")
    g.manual_seed(123)
    for call, n in enumerate((8192, 1000)):  # the limit (32 KiB) and an odd length
        ins = [torch.rand(n, device="cuda", generator=g) * 2 - 1 for _ in range(ws)]
        want = [torch.empty(n, device="cuda") for _ in range(ws)]
        world.allreduce(ins, want, algo="oneshot", scale=0.25)
        got = [torch.full((n,), float("nan"), device="cuda") for _ in range(ws)]
        torch.cuda.synchronize()
        code, msg = call_no_alloc(ins, got, 0.25)
        assert code == 0, msg
        for r in range(ws):
            torch.testing.assert_close(got[r], want[r], rtol=1e-6 * ws, atol=1e-6 * ws, msg=lambda m: f"call {call} rank {r}: {m}")
        ref = torch.stack([t.double() for t in ins]).sum(0) * 0.25
        torch.testing.assert_close(got[0].double(), ref, rtol=1e-6 * ws, atol=1e-6 * ws)


def test_no_alloc_entry_rejects_what_does_not_fit():
    ws = 2
    big = [torch.zeros(8193, device="cuda") for _ in range(ws)]
    code, msg = call_no_alloc(big, big, 1.0)
    assert code == 1 and "exceed the limit" in msg
    many = [torch.zeros(16, device="cuda") for _ in range(9)]
    code, msg = call_no_alloc(many, many, 1.0)
    assert code == 1 and "num_ranks" in msg


def test_no_alloc_entry_unaligned_eight_ranks_five_calls_in_place():
    # Buffers that are only 4-byte aligned (views at an odd element) take the element-wise path; 8 ranks;
    # five calls in a row alternate the two flag parities; the last call runs in place.
    ws = 8
    world = ar.EmuWorld(ws, 1 << 20, 1 << 20)
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    for call, n in enumerate((4097, 33, 8191, 1, 2500)):
        base_in = [torch.rand(n + 1, device="cuda", generator=g) * 2 - 1 for _ in range(ws)]
        ins = [t[1:] for t in base_in]
        want = [torch.empty(n + 1, device="cuda")[1:] for _ in range(ws)]
        if n >= ws:
            world.allreduce(ins, want, algo="oneshot", scale=0.125)
        ref = torch.stack([t.double() for t in ins]).sum(0) * 0.125
        in_place = call == 4
        got = ins if in_place else [torch.full((n + 3,), float("nan"), device="cuda")[3:] for _ in range(ws)]
        torch.cuda.synchronize()
        code, msg = call_no_alloc(ins, got, 0.125)
        assert code == 0, msg
        for r in range(ws):
            torch.testing.assert_close(got[r].double(), ref, rtol=1e-6 * ws, atol=1e-6 * ws, msg=lambda m: f"call {call} rank {r}: {m}")
            if n >= ws and not in_place:
                torch.testing.assert_close(got[r], want[r], rtol=1e-6 * ws, atol=1e-6 * ws)


def test_no_alloc_entry_empty_and_absurd_lengths():
    ws = 2
    bufs = [torch.ones(4, device="cuda") for _ in range(ws)]
    lib = _native.lib()
    fn = lib.ibcomm_emu_oneshot_allreduce_f32_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_float, C.c_void_p, C.c_char_p, C.c_size_t]
    ptrs = (C.c_void_p * ws)(*[t.data_ptr() for t in bufs])
    err = C.create_string_buffer(256)
    assert fn(ptrs, ptrs, ws, 0, 1.0, None, err, len(err)) == 0          # nothing to do, nothing launched
    for absurd in (1 << 62, (1 << 64) - 1):                              # would wrap when multiplied by 4
        assert fn(ptrs, ptrs, ws, absurd, 1.0, None, err, len(err)) == 1
        assert b"exceed the limit" in err.value
    torch.cuda.synchronize()
    assert all(torch.all(t == 1) for t in bufs)
