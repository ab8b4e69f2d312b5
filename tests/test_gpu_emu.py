"""Device kernels on one GPU: N ranks emulated in one cooperative launch
(EmuWorld).  Every result is compared with a plain PyTorch reference of the same
operation computed in fp64 (fp32 for integer types is exact anyway)."""
import pytest
import torch

import allreduce_proto_b200 as ar

pytestmark = pytest.mark.gpu

_worlds = {}


def world(ws, pool=0, work=0):
    key = (ws, pool, work)
    if key not in _worlds:
        _worlds[key] = ar.EmuWorld(ws, pool, work)
    return _worlds[key]


def make_inputs(ws, n, dtype, seed=0):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    if dtype in (torch.int32, torch.int64):
        return [torch.randint(-1000, 1000, (n,), device="cuda", dtype=dtype, generator=g) for _ in range(ws)]
    return [(torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dtype) for _ in range(ws)]


def reference(ins, scale, dtype):
    acc = torch.stack([t.double() for t in ins]).sum(0) * scale
    return acc


def tolerance(dtype, ws, wire=None):
    if dtype in (torch.int32, torch.int64):
        return 0.0, 0.0
    if dtype == torch.float64:
        return 1e-12, 1e-12
    if dtype == torch.float32 and wire is None:
        return 1e-6 * ws, 1e-6 * ws
    return 2e-2, 2e-2 * ws  # 16-bit storage or wire


def check(outs, want, dtype, ws, wire=None):
    rtol, atol = tolerance(dtype, ws, wire)
    for r, o in enumerate(outs):
        if dtype in (torch.int32, torch.int64):
            assert torch.equal(o.double(), want), f"rank {r}"
        else:
            torch.testing.assert_close(o.double(), want, rtol=rtol, atol=atol, msg=lambda m: f"rank {r}: {m}")


def test_native_library_is_loaded():
    world(2)
    with open("/proc/self/maps") as f:
        assert "libibcomm_cuda.so" in f.read()


@pytest.mark.parametrize("algo", ["ring", "rabenseifner"])
@pytest.mark.parametrize("ws", [2, 3, 4, 5, 6, 7, 8])
def test_program_algorithms_all_world_sizes(algo, ws):
    w = world(ws)
    for n in (ws, 2 * ws, 2521, 65536 + 3, 1 << 20):
        ins = make_inputs(ws, n, torch.float32, seed=n)
        outs = [torch.full((n,), float("nan"), device="cuda") for _ in range(ws)]
        w.allreduce(ins, outs, algo=algo)
        check(outs, reference(ins, 1.0, torch.float32), torch.float32, ws)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.int32, torch.int64, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("algo", ["ring", "rabenseifner", "oneshot"])
def test_dtypes(algo, dtype):
    ws = 4
    w = world(ws)
    for n in (1000, 32768):
        ins = make_inputs(ws, n, dtype, seed=7)
        outs = [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(ws)]
        w.allreduce(ins, outs, algo=algo)
        want = reference(ins, 1.0, dtype)
        if dtype in (torch.float16, torch.bfloat16):
            want = want.to(dtype).double() if algo == "oneshot" else want
        check(outs, want, dtype, ws)


@pytest.mark.parametrize("algo", ["ring", "rabenseifner", "oneshot"])
def test_scale_and_in_place(algo):
    ws = 8
    w = world(ws)
    n = 40000
    ins = make_inputs(ws, n, torch.float32, seed=3)
    want = reference(ins, 1.0 / ws, torch.float32)
    bufs = [t.clone() for t in ins]
    w.allreduce(bufs, None, algo=algo, scale=1.0 / ws)  # in place
    check(bufs, want, torch.float32, ws)


@pytest.mark.parametrize("algo", ["ring", "rabenseifner"])
@pytest.mark.parametrize("wire", [torch.bfloat16, torch.float16])
def test_wire_compression(algo, wire):
    ws = 4
    w = world(ws)
    n = 1 << 18
    ins = make_inputs(ws, n, torch.float32, seed=11)
    outs = [torch.zeros(n, device="cuda") for _ in range(ws)]
    w.allreduce(ins, outs, algo=algo, wire=wire, scale=0.25)
    check(outs, reference(ins, 0.25, torch.float32), torch.float32, ws, wire=wire)
    # every rank must hold the same bits
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("algo", ["ring", "rabenseifner"])
def test_small_staging_forces_slot_reuse(algo):
    # 1 MiB pool / work region with an 8 MiB message: chunks are cut to fit and
    # every staging slot is reused many times (credits).
    # Lengths that leave the last chunk shorter than the others: a slot then
    # holds chunks of different lengths over time.
    for ws in (4, 7):
        w = world(ws, 1 << 20, 1 << 20)
        for n in (2 << 20, (2 << 20) + 12345, 1000003):
            ins = make_inputs(ws, n, torch.float32, seed=5)
            outs = [torch.zeros(n, device="cuda") for _ in range(ws)]
            for channels in (1, 3, 8):
                w.allreduce(ins, outs, algo=algo, channels=channels)
                check(outs, reference(ins, 1.0, torch.float32), torch.float32, ws)


@pytest.mark.parametrize("ws", [2, 3, 4, 5, 8])
def test_direct_two_shot(ws):
    # The two-shot kernel with peer loads/stores (the code path of the NVLS
    # kernel minus multimem): in place on the ranks' buffers, and staged
    # through pool windows (1 MiB pool = 512 KiB windows, so 4 MiB messages
    # take several windows; the odd lengths end in a short last window).
    w = world(ws, 1 << 20, 1 << 20)
    for staged in (0, 1):
        w.set_direct_staging(staged)
        for n in (ws, 1000, 65536 + 3, 300001, 1 << 20, (1 << 20) + 12345):
            for dtype in (torch.float32, torch.bfloat16, torch.int32):
                ins = make_inputs(ws, n, dtype, seed=n + ws)
                want = reference(ins, 0.5 if dtype != torch.int32 else 1.0, dtype)
                outs = [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(ws)]
                w.allreduce(ins, outs, algo="direct", scale=0.5 if dtype != torch.int32 else 1.0)
                check(outs, want, dtype, ws)
        # in place
        bufs = make_inputs(ws, 50001, torch.float32, seed=3)
        want = reference(bufs, 1.0, torch.float32)
        w.allreduce(bufs, None, algo="direct")
        check(bufs, want, torch.float32, ws)
    w.set_direct_staging(0)


@pytest.mark.parametrize("split", [1, 0])
@pytest.mark.parametrize("ws", [2, 3, 4, 8])
def test_pipelined_staged_two_shot(ws, split):
    # The pipelined kernel for buffers that go through the pool (loader, reducer and storer warps on three
    # windows at once; the copy roles in blocks of their own, or, with the knob off, in every block).  2 MiB of
    # staging = four windows of 512 KiB, so the larger messages take many windows (the last one short); copies
    # by the bulk copy engine and, with the knob off, in registers.
    w = world(ws, 1 << 20, 1 << 20)
    w.set_direct_staging(2)
    ar.utils.set_tunable("IBCOMM_STAGED_SPLIT", split)
    try:
        for tma in (1, 0):
            ar.utils.set_tunable("IBCOMM_STAGED_TMA", tma)
            for dtype in (torch.float32, torch.bfloat16, torch.int32, torch.float64):
                for n in (8 * ws, 4096, 65536 + 8, 300000, 1 << 20, (1 << 20) + 12344):
                    ins = make_inputs(ws, n, dtype, seed=n + ws)
                    scale = 0.5 if dtype != torch.int32 else 1.0
                    want = reference(ins, scale, dtype)
                    outs = [torch.zeros(n, device="cuda", dtype=dtype) for _ in range(ws)]
                    for channels in ((0,) if n < (1 << 20) else (0, 1, 3)):
                        w.allreduce(ins, outs, algo="direct", scale=scale, channels=channels)
                        check(outs, want, dtype, ws)
            # in place, several calls back to back without a host synchronisation in between
            bufs = make_inputs(ws, 500000, torch.float32, seed=3)
            want = reference(bufs, 1.0, torch.float32)
            w.allreduce(bufs, None, algo="direct")
            check(bufs, want, torch.float32, ws)
            ins = make_inputs(ws, 700000, torch.float32, seed=4)
            outs = [torch.zeros(700000, device="cuda") for _ in range(ws)]
            for _ in range(5):
                w.allreduce(ins, outs, algo="direct", sync=False)
            torch.cuda.synchronize()
            check(outs, reference(ins, 1.0, torch.float32), torch.float32, ws)
    finally:
        ar.utils.set_tunable("IBCOMM_STAGED_TMA", -1)
        ar.utils.set_tunable("IBCOMM_STAGED_SPLIT", -1)
        w.set_direct_staging(0)


@pytest.mark.parametrize("shape", [(6, 3, 2, 3, 1), (4, 2, 3, 2, 0), (6, 4, 2, 2, 1), (3, 1, 1, 1, 1)])
@pytest.mark.parametrize("ws", [2, 4])
def test_pipelined_staged_groups_and_posters(ws, shape):
    # Split mode with several groups per role (window k belongs to group k mod groups, each group with flag
    # rows of its own) and poster warps behind the reducer groups; many short windows so that every group
    # takes several, the last one short.
    bufs, lg, rg, sg, posters = shape
    knobs = {"IBCOMM_STAGED_SPLIT": 1, "IBCOMM_STAGED_BUFFERS": bufs, "IBCOMM_STAGED_LOAD_GROUPS": lg,
             "IBCOMM_STAGED_REDUCE_GROUPS": rg, "IBCOMM_STAGED_STORE_GROUPS": sg, "IBCOMM_STAGED_POSTERS": posters}
    w = world(ws, 1 << 20, 1 << 20)
    w.set_direct_staging(2)
    for k, v in knobs.items():
        ar.utils.set_tunable(k, v)
    try:
        for tma in (1, 0):
            ar.utils.set_tunable("IBCOMM_STAGED_TMA", tma)
            for n in (8 * ws, 65536 + 8, (1 << 20) + 12344, 3 << 20):
                ins = make_inputs(ws, n, torch.float32, seed=n + ws)
                outs = [torch.zeros(n, device="cuda") for _ in range(ws)]
                for _ in range(2):  # back to back, no host synchronisation in between
                    w.allreduce(ins, outs, algo="direct", scale=0.25, sync=False)
                torch.cuda.synchronize()
                check(outs, reference(ins, 0.25, torch.float32), torch.float32, ws)
        ins = make_inputs(ws, 1 << 20, torch.float32, seed=9)
        outs = [torch.zeros(1 << 20, device="cuda") for _ in range(ws)]
        w.allreduce(ins, outs, algo="direct", wire=torch.bfloat16)
        check(outs, reference(ins, 1.0, torch.float32), torch.float32, ws, wire=torch.bfloat16)
    finally:
        for k in list(knobs) + ["IBCOMM_STAGED_TMA"]:
            ar.utils.set_tunable(k, -1)
        w.set_direct_staging(0)


@pytest.mark.parametrize("split", [1, 0])
@pytest.mark.parametrize("wire", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ws", [2, 4, 8])
def test_two_shot_with_16_bit_wire(ws, wire, split):
    # fp32 buffers, 16-bit values in the pool and on the wire, fp32 sums: the direct two-shot through the
    # pipelined kernel.  Every rank must end up with the same bits.
    w = world(ws, 1 << 20, 1 << 20)
    ar.utils.set_tunable("IBCOMM_STAGED_SPLIT", split)
    try:
        for n in (8 * ws, 65536, 300000, (1 << 20) + 8):
            ins = make_inputs(ws, n, torch.float32, seed=n)
            outs = [torch.zeros(n, device="cuda") for _ in range(ws)]
            w.allreduce(ins, outs, algo="direct", wire=wire, scale=1.0 / ws)
            check(outs, reference(ins, 1.0 / ws, torch.float32), torch.float32, ws, wire=wire)
            for o in outs[1:]:
                assert torch.equal(o, outs[0])
    finally:
        ar.utils.set_tunable("IBCOMM_STAGED_SPLIT", -1)


@pytest.mark.parametrize("split", [1, 0])
def test_pipelined_staged_wait_runs_out(split):
    # A rank that takes no part: the others' loaders, reducers and storers give up after the limit, the kernel
    # returns, the status names the wait, and the world stays usable.
    ws = 4
    w = ar.EmuWorld(ws, 1 << 20, 1 << 20)
    w.set_direct_staging(2)
    w.set_timeout_ms(200)
    ar.utils.set_tunable("IBCOMM_STAGED_SPLIT", split)
    try:
        n = 1 << 16
        ins = make_inputs(ws, n, torch.float32)
        outs = [torch.zeros(n, device="cuda") for _ in range(ws)]
        w.set_silent_rank(1)
        with pytest.raises(ar.IbcommError) as e:
            w.allreduce(ins, outs, algo="direct")
        assert e.value.code == ar.TRANSPORT_ERROR
        assert w.last_status()["code"] in (1, 2)
        w.set_silent_rank(-1)
        w.set_timeout_ms(5000)
        w.allreduce(ins, outs, algo="direct")
        check(outs, reference(ins, 1.0, torch.float32), torch.float32, ws)
    finally:
        ar.utils.set_tunable("IBCOMM_STAGED_SPLIT", -1)


def test_unaligned_buffers_take_the_scalar_path():
    ws = 3
    w = world(ws)
    n = 5000
    base = make_inputs(ws, n + 1, torch.float32, seed=9)
    ins = [t[1:] for t in base]  # 4-byte aligned only
    outs_base = [torch.zeros(n + 3, device="cuda") for _ in range(ws)]
    outs = [t[3:] for t in outs_base]
    for algo in ("ring", "rabenseifner", "oneshot", "direct"):
        w.allreduce(ins, outs, algo=algo)
        check(outs, reference(ins, 1.0, torch.float32), torch.float32, ws)


def test_repeated_calls_mixed_algorithms():
    ws = 8
    w = world(ws)
    n = 50000
    ins = make_inputs(ws, n, torch.float32, seed=1)
    outs = [torch.zeros(n, device="cuda") for _ in range(ws)]
    want = reference(ins, 1.0, torch.float32)
    for it in range(30):
        algo = ("ring", "oneshot", "rabenseifner", "direct")[it % 4]
        w.allreduce(ins, outs, algo=algo, sync=False)
    torch.cuda.synchronize()
    check(outs, want, torch.float32, ws)


def test_error_codes():
    w = world(2)
    a = [torch.zeros(1, device="cuda") for _ in range(2)]
    with pytest.raises(ar.IbcommError) as e:
        w.allreduce(a, None, algo="ring")
    assert e.value.code == ar.NOT_SUPPORTED  # fewer elements than ranks
    big = [torch.zeros((16 << 20) // 4 + 4, device="cuda") for _ in range(2)]  # one vector more than a two-rank slot holds
    with pytest.raises(ar.IbcommError) as e:
        w.allreduce(big, None, algo="oneshot")
    assert e.value.code == ar.INVALID_ARGUMENT  # beyond the one-shot slot
    with pytest.raises(ar.IbcommError) as e:
        w.allreduce(big, None, algo="nvls")
    assert e.value.code == ar.NOT_SUPPORTED


def test_bounded_wait_reports_timeout():
    # One rank does not take part: the others' waits run out after the limit,
    # the kernel returns, the status says who was missing, and the world stays usable.
    ws = 4
    w = ar.EmuWorld(ws, 1 << 20, 1 << 20)
    w.set_timeout_ms(200)
    n = 4096
    ins = make_inputs(ws, n, torch.float32)
    outs = [torch.zeros(n, device="cuda") for _ in range(ws)]
    w.set_silent_rank(2)
    with pytest.raises(ar.IbcommError) as e:
        w.allreduce(ins, outs, algo="ring")
    assert e.value.code == ar.TRANSPORT_ERROR
    st = w.last_status()
    assert st["code"] in (1, 2) and st["kind"] == 1  # timeout (or peer abort) at the entry barrier
    w.set_silent_rank(-1)
    w.set_timeout_ms(5000)
    w.allreduce(ins, outs, algo="ring")
    check(outs, reference(ins, 1.0, torch.float32), torch.float32, ws)


@pytest.mark.parametrize("ws", [2, 3, 5, 8])
def test_reduce_scatter_and_all_gather(ws):
    # The halves of the two-shot allreduce as collectives: in place on the
    # ranks' buffers and through pool windows (1 MiB pool, so the larger
    # blocks take several windows, the last one short); blocks of whole
    # 16-byte vectors and ragged ones (element units); every element type.
    w = world(ws, 1 << 20, 1 << 20)
    for staged in (0, 1):
        w.set_direct_staging(staged)
        for m in (1, 37, 4096, 100000 // ws * 4, 70001):
            for dtype in (torch.float32, torch.bfloat16, torch.int32, torch.float64):
                ins = make_inputs(ws, m * ws, dtype, seed=m + ws)
                scale = 0.5 if dtype not in (torch.int32,) else 1.0
                want = reference(ins, scale, dtype)
                outs = [torch.zeros(m, device="cuda", dtype=dtype) for _ in range(ws)]
                w.reduce_scatter(ins, outs, scale=scale)
                for r in range(ws):
                    check([outs[r]], want[r * m:(r + 1) * m], dtype, ws)
                gathered = [torch.zeros(m * ws, device="cuda", dtype=dtype) for _ in range(ws)]
                w.all_gather(outs, gathered)
                whole = torch.cat(outs)
                for r in range(ws):
                    assert torch.equal(gathered[r], whole), f"all-gather rank {r} m={m} {dtype}"
        # element-aligned user buffers (odd offset) in vector-sized blocks
        m = 4096
        ins = [t[1:] for t in make_inputs(ws, m * ws + 1, torch.float32, seed=5)]
        outs = [torch.zeros(m + 1, device="cuda")[1:] for _ in range(ws)]
        w.reduce_scatter(ins, outs)
        want = reference(ins, 1.0, torch.float32)
        for r in range(ws):
            check([outs[r]], want[r * m:(r + 1) * m], torch.float32, ws)
        gathered = [torch.zeros(m * ws + 1, device="cuda")[1:] for _ in range(ws)]
        w.all_gather(outs, gathered)
        for r in range(ws):
            assert torch.equal(gathered[r], torch.cat(outs))
    w.set_direct_staging(0)


def test_executor_self_check_reports_bad_program():
    # A rank whose ops do not fit the message it was given stops at the bounds
    # check of its first op (before any access), reports "bad program" and
    # tells the others to stop; the world stays usable.
    ws = 4
    w = ar.EmuWorld(ws, 1 << 20, 1 << 20)
    w.set_timeout_ms(2000)
    n = 8192
    ins = make_inputs(ws, n, torch.float32)
    outs = [torch.zeros(n, device="cuda") for _ in range(ws)]
    w.set_bad_program_rank(1)
    with pytest.raises(ar.IbcommError) as e:
        w.allreduce(ins, outs, algo="ring")
    assert e.value.code == ar.TRANSPORT_ERROR
    assert "bad program" in str(e.value)
    st = w.last_status()
    assert st["code"] == 3 and st["rank"] == 1 and st["op_index"] == 0
    w.set_bad_program_rank(-1)
    w.allreduce(ins, outs, algo="rabenseifner")
    check(outs, reference(ins, 1.0, torch.float32), torch.float32, ws)


def test_world_size_one_copy_scale_kernel():
    comm = ar.Communicator(1, 0)
    for n in (1, 5, 4096, (1 << 20) + 7):
        x = torch.randn(n, device="cuda")
        y = torch.empty_like(x)
        comm.allreduce(x, y, scale=0.5, sync=True)
        torch.testing.assert_close(y, x * 0.5)
    # The halves at world size 1 are the same copy (the reduce-scatter with its scale).
    x = torch.randn(4099, device="cuda")
    y = torch.empty_like(x)
    comm.reduce_scatter(x, y, scale=0.25, sync=True)
    torch.testing.assert_close(y, x * 0.25)
    z = torch.empty_like(x)
    comm.all_gather(y, z, sync=True)
    torch.testing.assert_close(z, y)
    x = torch.randn(100003, device="cuda")
    for out_dtype in (torch.bfloat16, torch.float16):
        y = ar.ops.copy_scale(x, scale=2.0, out_dtype=out_dtype)
        torch.testing.assert_close(y, (x * 2.0).to(out_dtype))
    z = ar.ops.copy_scale(x[1:], scale=3.0)  # unaligned -> plain kernel
    torch.testing.assert_close(z, x[1:] * 3.0)


def test_gradient_buckets_single_process():
    from allreduce_proto_b200.models import resnet50_param_shapes, synthetic_grads
    shapes = [s for _, s in resnet50_param_shapes()]
    comm = ar.Communicator(1, 0)
    buckets = ar.GradientBuckets(shapes, comm=comm, bucket_bytes=25 << 20)
    assert buckets.num_buckets == 5
    grads = synthetic_grads("cuda")
    buckets.load(grads)
    buckets.allreduce(average=True, sync=True)
    for v, g in zip(buckets.views, grads):
        torch.testing.assert_close(v, g)


def test_tester_binary_emulated(bins):
    import subprocess
    for algo in ("ring", "rabenseifner"):
        for np_ in (2, 3, 4, 5, 8):
            p = subprocess.run([bins["allreduce_tester"], "--emulate", str(np_), algo, "64k", "i*np+p", "i*np*np+np*(np-1)/2"],
                               stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
            assert p.returncode == 0, p.stderr
    # chunk-size validation and short vectors exit with the reference's codes
    import os
    env = dict(os.environ, IBCOMM_CHUNKSIZE="3")
    p = subprocess.run([bins["allreduce_tester"], "--emulate", "4", "ring", "1k", "1", "np"], env=env, stderr=subprocess.PIPE)
    assert p.returncode == 1
    p = subprocess.run([bins["allreduce_tester"], "--emulate", "2", "ring", "4", "1", "np"], stderr=subprocess.PIPE)
    assert p.returncode == 4


def _tester(bins, args, env=None, timeout=600):
    import os
    import subprocess
    p = subprocess.run([bins["allreduce_tester"], *args], env=dict(os.environ, **(env or {})), stdout=subprocess.PIPE,
                       stderr=subprocess.PIPE, text=True, timeout=timeout)
    return p.returncode, p.stderr


def test_chunk_size_on_the_device_path(bins):
    # The reference's chunk-size cases (tests/allreduce_test.py:180-225) on device buffers: 4 emulated ranks,
    # 1 KiB of ints, IBCOMM_CHUNKSIZE 4..128 bytes -> 0; 0..3, -128 and "1k" -> invalid argument.
    for algo in ("ring", "rabenseifner"):
        for chunk in (4, 8, 16, 32, 64, 128):
            code, err = _tester(bins, ["--emulate", "4", algo, "1k", "i*np+p", "i*np*np+np*(np-1)/2"], {"IBCOMM_CHUNKSIZE": str(chunk)})
            assert code == 0, (algo, chunk, err)
    for chunk in ("0", "1", "2", "3", "-128", "1k"):
        code, _ = _tester(bins, ["--emulate", "4", "ring", "1k", "1", "np"], {"IBCOMM_CHUNKSIZE": chunk})
        assert code == ar.INVALID_ARGUMENT, chunk


@pytest.mark.parametrize("algo", ["rabenseifner", "ring"])
def test_staging_offsets_that_are_not_vector_aligned(algo):
    # Short messages cut chunk boundaries at arbitrary elements: a range can then be 16-byte aligned in the
    # user buffer and not in the (narrower) staging slot, or the other way round; such slices take the
    # element-by-element path.  Lengths and views chosen to hit both.
    for ws in (3, 4):
        w = world(ws)
        for wire in (torch.bfloat16, torch.float16):
            for n in (1000, 2521):
                ins = make_inputs(ws, n, torch.float32, seed=n)
                outs = [torch.zeros(n, device="cuda") for _ in range(ws)]
                w.allreduce(ins, outs, algo=algo, wire=wire)
                check(outs, reference(ins, 1.0, torch.float32), torch.float32, ws, wire=wire)
        base = make_inputs(ws, 2521 + 4, torch.float16, seed=2)
        ins = [t[4:] for t in base]  # 8-byte offset in a 16-bit type
        outs = [torch.zeros(2521 + 4, device="cuda", dtype=torch.float16)[4:] for _ in range(ws)]
        w.allreduce(ins, outs, algo=algo)
        check(outs, reference(ins, 1.0, torch.float16), torch.float16, ws)


@pytest.mark.slow
def test_aging_on_the_device_path(bins):
    # The reference's ageing case (tests/allreduce_test.py:227-235): 100 ring and 100 Rabenseifner allreduces
    # back to back on device buffers, 4 ranks (emulated here; 32 MiB each).
    for algo in ("ring", "rabenseifner"):
        code, err = _tester(bins, ["--emulate", "4", "--iters", "100", algo, "32M", "i*np+p", "i*np*np+np*(np-1)/2"])
        assert code == 0, (algo, err)


def test_staging_pool_with_pinned_blocks_and_cuda_streams(bins):
    # include/ibcomm/memory_pool.h under USE_CUDA: the exclusive controller hands out pinned slots paired with
    # real streams, grows by a block and by streams when six slots are out at once (tests/cpp/threads_test.cpp).
    import subprocess
    p = subprocess.run(["timeout", "120s", bins["threads_test_cuda"], "pool"], stdout=subprocess.PIPE,
                       stderr=subprocess.PIPE, text=True)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "pool OK" in p.stdout
