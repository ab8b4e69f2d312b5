"""Host utilities: the C++ unit-test binary (size parser tables, power-of-two
gate, partitioner, expression compiler, error policy — the reference's
tests/unittest.cpp cases and more) and the same functions through the Python
package."""
import subprocess

import pytest

import allreduce_proto_b200 as ar
from allreduce_proto_b200 import utils


def test_cpp_unittest_binary(bins):
    p = subprocess.run([bins["unittest"]], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert p.returncode == 0, p.stdout


def test_parse_number_tables():
    for sign in ("", "-", "+"):
        for suffix in ("", "b", "B", "k", "kb", "K", "m", "mb", "M", "g", "gb", "G"):
            assert utils.parse_number(f"{sign}0{suffix}") == 0
    assert utils.parse_number("1k") == 1024
    assert utils.parse_number("31kb") == 31 * 1024
    assert utils.parse_number("713m") == 713 * 1024 * 1024
    assert utils.parse_number("128M") == 128 << 20
    for bad in ("0.5", "a", "b", "B", "0x", "97MiB", ""):
        with pytest.raises(ValueError):
            utils.parse_number(bad)


def test_get_exp_of_two():
    assert [utils.get_exp_of_two(n) for n in (0, 1, 2, 128, 127, 129)] == [0, 0, 1, 7, 0, 0]


def test_split_buffer_and_blocks():
    r = utils.split_buffer(1000, 4, 4)
    assert len(r) == 16 and r[0] == (0, 63) and r[-1][1] == 1000
    assert all(r[i][0] == r[i - 1][1] for i in range(1, len(r)))
    assert len(utils.split_buffer(4, 4, 2)) == 4  # empty tail ranges dropped
    assert utils.rank_to_chunk(16, 4, 1) == [4, 5, 6, 7]
    assert [len(utils.rank_to_chunk(10, 4, r)) for r in range(4)] == [3, 3, 2, 2]


def test_split_buffer_error_codes():
    def code(*a):
        try:
            utils.split_buffer(*a)
        except ar.IbcommError as e:
            return e.code
        return 0
    assert code(1, 4, 2) == ar.NOT_SUPPORTED            # shorter than the world size
    assert code(256, 4, 4, 3) == ar.INVALID_ARGUMENT    # not a multiple of sizeof(T)
    assert code(256, 4, 4, 1024) == ar.INVALID_ARGUMENT  # fewer than 2 * ws chunks
    assert code(256, 4, 4, 128) == 0
    assert code(1, 4, 2, 3) == ar.NOT_SUPPORTED         # the length is checked first


def test_ring_program_shape():
    # rank 1 of 4: first op sends its own block's highest chunk from sendbuf;
    # every op that stores locally with a remote store too is a forward.
    ops = utils.describe_program("ring", 1, 4, 4096)
    assert ops[0].startswith("[1792+256] a=send")
    assert sum("remote" in o for o in ops) == sum(1 for o in ops) - 4  # last all-gather block is not forwarded
    # Rabenseifner on 3 ranks folds ranks 0 and 1: rank 0 ends by receiving everything.
    ops0 = utils.describe_program("rabenseifner", 0, 3, 4096)
    assert "remote" not in ops0[-1] and "local" in ops0[-1]


def test_bandwidth_helpers():
    assert utils.busbw_gbs(1 << 30, 1.0, 8) == pytest.approx((1 << 30) / 1e9 * 1.75)
    assert utils.busbw_gbs(1 << 30, 1.0, 1) == pytest.approx((1 << 30) / 1e9)
    assert utils.ring_bytes_per_gpu(256 << 20, 8) == pytest.approx(2 * (256 << 20) * 7 / 8)
    assert utils.nvls_bytes_per_gpu(256 << 20, 8) == pytest.approx((256 << 20) * 1.125)


def test_resnet50_shapes():
    from allreduce_proto_b200.models import resnet50_num_params, resnet50_param_shapes
    assert resnet50_num_params() == 25_557_032
    assert len(resnet50_param_shapes()) == 161
    plan = ar.plan_buckets([100, 200, 50, 1000], 4, 1024)
    assert plan == [[0], [1, 2], [3]]


def test_python_api_argument_checks():
    # A world of one rank needs no peers: the host paths and the argument checks run in-process.
    import torch

    import allreduce_proto_b200 as ar
    comm = ar.Communicator(1, 0)
    x = torch.arange(12, dtype=torch.float32)
    y = torch.empty(12)
    comm.allreduce(x, y, scale=0.5)
    assert torch.equal(y, x * 0.5)
    comm.reduce_scatter(x, y, scale=2.0)          # one rank: one block
    assert torch.equal(y, x * 2.0)
    z = torch.empty(12)
    comm.all_gather(y, z)
    assert torch.equal(z, y)
    with pytest.raises(ar.IbcommError) as e:
        comm.reduce_scatter(x, torch.empty(5))    # not world_size blocks
    assert e.value.code == ar.INVALID_ARGUMENT
    with pytest.raises(ar.IbcommError) as e:
        comm.all_gather(x, torch.empty(12, dtype=torch.float64))
    assert e.value.code == ar.INVALID_ARGUMENT
    with pytest.raises(ar.IbcommError):
        comm.allreduce(x, torch.empty(11))
    with pytest.raises(ValueError):
        comm.register(x)                          # registration is for CUDA tensors
    assert comm.staged_timeline() == {"windows": 0, "reduce": [], "load": [], "store": []}   # nothing traced
    ar.utils.set_tunable("IBCOMM_STAGED_BUFFERS", 5)
    assert ar.utils.get_tunable("IBCOMM_STAGED_BUFFERS", 3) == 5
    ar.utils.set_tunable("IBCOMM_STAGED_BUFFERS", -1)
    assert ar.utils.get_tunable("IBCOMM_STAGED_BUFFERS", 3) == 3
    comm.close()


def test_gradient_buckets_without_a_communicator():
    import torch

    import allreduce_proto_b200 as ar
    shapes = [(3, 5), (7,), (2, 2, 2)]
    b = ar.GradientBuckets(shapes, device="cpu", bucket_bytes=64, shardable=True)
    assert b.num_buckets >= 2 and [tuple(v.shape) for v in b.views] == shapes
    b.load([torch.full(s, 2.0) for s in shapes])
    b.allreduce(average=True)                     # no communicator: a plain scale by 1/1
    assert all(torch.equal(v, torch.full(s, 2.0)) for v, s in zip(b.views, shapes))
    assert [s.numel() for s in b.reduce_scatter()] == [f.numel() for f in b.flat]
    b.all_gather()
    with pytest.raises(ValueError):
        ar.GradientBuckets(shapes, device="cpu").shards()


def test_algorithm_table():
    # The choices `auto` makes (measured on 2, 4 and 8 B200); needs no GPU.
    from allreduce_proto_b200.utils import choose_algorithm as ca
    MiB = 1 << 20
    assert ca(4096, 8)[0] == "oneshot"
    assert ca(256 * MiB, 8) == ("nvls", 64)                      # symmetric buffers: reduce in the switch
    assert ca(256 * MiB, 4)[0] == "nvls"
    assert ca(256 * MiB, 2)[0] == "direct"                       # two ranks: 1.0 S per direction beats 1.5 S
    assert ca(256 * MiB, 8, nvls=False)[0] == "direct"           # registered buffers, or no multicast
    assert ca(256 * MiB, 8, mapped=False)[0] == "nvls"           # ordinary buffers: through the pool, pipelined in the kernel
    assert ca(256 * MiB, 8, nvls=False, mapped=False)[0] == "rabenseifner"   # no switch, power-of-two ranks
    assert ca(256 * MiB, 6, nvls=False, mapped=False)[0] == "ring"
    assert ca(8 * MiB, 8, mapped=False)[0] == "nvls"
    assert ca(256 << 10, 8, mapped=False)[0] == "oneshot"
    assert ca(4 * MiB, 2, mapped=False)[0] == "oneshot"          # two ranks: one push each is all the traffic there is
    assert ca(2 * MiB, 2)[0] == "oneshot" and ca(8 * MiB, 2)[0] == "direct"
    assert ca(64 * MiB, 2, mapped=False)[0] == "ring"            # two ranks: the ring is one exchange each way
    assert ca(16 * MiB, 4, nvls=False, mapped=False)[0] == "direct"   # staged and pipelined inside the kernel
    assert ca(256 * MiB, 2, mapped=False)[0] == "ring"
    for ws in range(2, 9):
        for nb in (4, 4096, MiB, 64 * MiB, 1 << 30):
            for nvls in (False, True):
                for mapped in (False, True):
                    algo, ch = ca(nb, ws, nvls=nvls, mapped=mapped)
                    assert algo in ("oneshot", "nvls", "direct", "ring", "rabenseifner") and 1 <= ch <= 256
                    assert nvls or algo != "nvls"
                    assert ca(nb, ws, nvls=nvls, mapped=mapped, max_channels=8)[1] <= 8


def test_c_headers_compile_as_c99(tmp_path, bins):
    # The C API is the surface other languages bind to: plain C, no C++ in the headers,
    # and the library exports what the header declares.
    import shutil
    import subprocess
    from pathlib import Path
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    root = Path(__file__).resolve().parent.parent
    src = tmp_path / "t.c"
    src.write_text('#include "ibcomm/c_api.h"\n#include "ibcomm/no_alloc.h"\n#include <stdio.h>\n'
                   'int main(void) { int a = 0, c = 0;\n'
                   '  int rc = ibcomm_choose_algorithm((size_t)256 << 20, 8, 1, 1, 0, &a, &c);\n'
                   '  printf("%d %d %d\\n", rc, a, c); return rc; }\n')
    lib_dir = root / "allreduce_proto_b200" / "_lib"
    exe = tmp_path / "t"
    b = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", f"-I{root / 'include'}", str(src),
                        f"-L{lib_dir}", "-libcomm", f"-Wl,-rpath,{lib_dir}", "-o", str(exe)],
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert b.returncode == 0, b.stdout
    p = subprocess.run([str(exe)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert p.returncode == 0 and p.stdout.split() == ["0", "3", "64"], p.stdout   # nvls, 64 channels


def test_numa_helper_is_a_no_op_without_a_gpu():
    from allreduce_proto_b200.utils import device_numa_node, numa
    assert numa._parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert numa._parse_cpulist("") == set()
    import os
    before = os.sched_getaffinity(0)
    with device_numa_node(0) as node:
        assert node is None or isinstance(node, int)
    assert os.sched_getaffinity(0) == before


def test_bench_reference_arm_prints_unavailable():
    # The reference cannot be built on this image (no libibverbs, no MPI): the arm says so in one JSON line, exit 0.
    import json
    import subprocess
    import sys
    from pathlib import Path
    bench = str(Path(__file__).resolve().parent.parent / "bench.py")
    p = subprocess.run([sys.executable, bench, "--impl", "reference", "--gpus", "8", "--steps", "5", "--warmup", "3"],
                       stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    assert p.returncode == 0, p.stderr
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and "\n" not in line["unavailable"]


def test_closed_communicator_raises_instead_of_crashing():
    import torch

    import allreduce_proto_b200 as ar
    comm = ar.Communicator(1, 0)
    comm.close()
    comm.close()  # closing twice is fine
    for call in (comm.barrier, lambda: comm.allreduce(torch.ones(4)), lambda: comm.set_timeout_ms(5)):
        with pytest.raises(ar.IbcommError) as e:
            call()
        assert e.value.code == ar.INVALID_ARGUMENT


def test_partitioner_properties():
    # Property test (hypothesis): whatever the length, element size, world size and chunk size, the chunks
    # tile [0, n) without gaps or overlaps, there are at least as many chunks as ranks want, blocks of
    # chunk ids are contiguous and cover every chunk once.
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=300, deadline=None)
    @given(n=st.integers(1, 1 << 22), esize=st.sampled_from([1, 2, 4, 8]), ws=st.integers(1, 8),
           chunk_elems=st.integers(0, 1 << 16))
    def check(n, esize, ws, chunk_elems):
        chunk_bytes = chunk_elems * esize
        try:
            r = utils.split_buffer(n, esize, ws, chunk_bytes)
        except ar.IbcommError as e:
            assert e.code in (ar.INVALID_ARGUMENT, ar.NOT_SUPPORTED)
            if n < ws:
                assert e.code == ar.NOT_SUPPORTED
            return
        assert n >= ws
        assert r[0][0] == 0 and r[-1][1] == n
        assert all(b < e for b, e in r)
        assert all(r[i][0] == r[i - 1][1] for i in range(1, len(r)))
        if chunk_bytes > 0:
            assert all(e - b <= chunk_elems for b, e in r)
            assert len(r) >= 2 * ws or ws == 1
        else:
            assert len(r) <= 4 * ws
        owned = [utils.rank_to_chunk(len(r), ws, k) for k in range(ws)]
        flat = [c for o in owned for c in o]
        assert flat == list(range(len(r)))
        assert max(len(o) for o in owned) - min(len(o) for o in owned) <= 1

    check()
