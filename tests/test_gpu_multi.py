"""Multi-GPU tests: one process per GPU over real peer mappings (and NVSwitch
multicast where the box has it).  Skipped on machines with one GPU, where the
same kernels are covered by the emulated ranks of test_gpu_emu.py."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

WORKER = str(Path(__file__).resolve().parent / "multigpu_worker.py")
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0
needs2 = pytest.mark.skipif(NGPU < 2, reason="needs at least two GPUs")


def run(bins, np, case, env=None, timeout=300):
    cmd = ["timeout", f"{timeout}s", bins["ibcomm_run"], "-np", str(np)]
    for k, v in (env or {}).items():
        cmd += ["-x", f"{k}={v}"]
    cmd += [sys.executable, WORKER, case]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    return p.returncode, p.stderr[-4000:]


def world_sizes():
    return [n for n in (2, 3, 4, 5, 6, 7, 8) if n <= NGPU]


@needs2
@pytest.mark.parametrize("np_", world_sizes())
def test_allreduce_every_algorithm(bins, np_):
    code, err = run(bins, np_, "allreduce")
    assert code == 0, err


@needs2
@pytest.mark.parametrize("np_", [n for n in (2, 4, 8) if n <= NGPU])
def test_symmetric_zero_copy(bins, np_):
    code, err = run(bins, np_, "symmetric")
    assert code == 0, err


@needs2
def test_ranks_as_threads_of_one_process(bins):
    # One process, one host thread and one communicator per GPU.
    np_ = min(NGPU, 4)
    p = subprocess.run(["timeout", "300s", bins["threads_test_cuda"], "cuda", str(np_)], stdout=subprocess.PIPE,
                       stderr=subprocess.PIPE, text=True, env={**os.environ, "IBCOMM_TIMEOUT_MS": "5000"})
    assert p.returncode == 0, p.stderr[-2000:]
    assert "threads_test OK" in p.stdout


@needs2
@pytest.mark.parametrize("np_", [n for n in (2, 3, 8) if n <= NGPU])
def test_reduce_scatter_and_all_gather(bins, np_):
    code, err = run(bins, np_, "rsag")
    assert code == 0, err


@needs2
def test_sharded_gradient_buckets(bins):
    code, err = run(bins, min(NGPU, 4), "sharded_buckets")
    assert code == 0, err


@needs2
def test_registered_user_buffers(bins):
    code, err = run(bins, min(NGPU, 4), "registered")
    assert code == 0, err


@needs2
@pytest.mark.parametrize("np_", sorted({min(NGPU, 2), min(NGPU, 8)}))
def test_registered_buffers_bound_to_the_switch(bins, np_):
    # Registration binds ordinary tensors to the NVSwitch multicast where the driver allows it; the switch
    # kernel then works on them in place.  Results are checked either way.
    code, err = run(bins, np_, "registered_switch")
    assert code == 0, err


@needs2
def test_staged_buffers_over_several_windows(bins):
    code, err = run(bins, min(NGPU, 4), "staged")
    assert code == 0, err


@needs2
def test_without_multicast_and_with_ipc_handles(bins):
    code, err = run(bins, 2, "allreduce", env={"IBCOMM_DISABLE_NVLS": "1"})
    assert code == 0, err
    code, err = run(bins, 2, "allreduce", env={"IBCOMM_ARENA_MODE": "ipc"})
    assert code == 0, err


@needs2
def test_device_send_recv_bcast(bins):
    code, err = run(bins, min(NGPU, 4), "sendrecv")
    assert code == 0, err


@needs2
def test_resnet50_gradient_buckets(bins):
    code, err = run(bins, min(NGPU, 8), "buckets")
    assert code == 0, err


@needs2
def test_rank_leaving_is_detected(bins):
    # NVLS off: a rank that exits while bound to a multicast object can raise
    # NVLink faults on its peers; plain peer mappings do not.
    code, err = run(bins, 2, "leave", env={"IBCOMM_DISABLE_NVLS": "1", "NCCL_NVLS_ENABLE": "0"})
    assert code == 0, err


@needs2
def test_cuda_graph_capture_and_replay(bins):
    code, err = run(bins, 2, "graph")
    assert code == 0, err


@needs2
def test_device_trace(bins, tmp_path):
    prefix = str(tmp_path / "devtrace")
    code, err = run(bins, 2, "trace", env={"IBCOMM_TRACE": "1", "IBCOMM_TRACE_FILE": prefix})
    assert code == 0, err
    for r in range(2):
        lines = {ln.split(",")[0]: ln.split(",")[1:] for ln in Path(f"{prefix}_{r}.dat").read_text().splitlines()}
        # begin/duration pairs of the kernel's waits ("received") and data phases ("reduced"), and of the host's launches
        assert len([v for v in lines["received"] if v]) >= 4
        assert len([v for v in lines["reduced"] if v]) >= 4
        assert len([v for v in lines["issue_redu_kernel"] if v]) >= 2
        assert all(float(v) >= 0 for v in lines["reduced"] if v)


@needs2
def test_tester_binary_on_gpus(bins):
    for algo in ("ring", "rabenseifner"):
        cmd = ["timeout", "120s", bins["ibcomm_run"], "-np", "2", bins["allreduce_tester"], "--device", "cuda", algo, "128M",
               "i*np+p", "i*np*np+np*(np-1)/2"]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        assert p.returncode == 0, p.stderr[-2000:]


@needs2
@pytest.mark.parametrize("np_", [n for n in (2, 4, 8) if n <= NGPU])
def test_pipelined_staged_two_shot(bins, np_):
    # Ordinary buffers through the pipelined kernel (switch and direct), several windows, 16-bit wire.
    code, err = run(bins, np_, "pipelined")
    assert code == 0, err


@needs2
@pytest.mark.parametrize("np_", [n for n in (2, 4, 8) if n <= NGPU])
def test_hybrid_switch_plus_direct(bins, np_):
    code, err = run(bins, np_, "hybrid")
    assert code == 0, err


@needs2
def test_device_send_recv_errors_leave_the_communicator_usable(bins):
    # A receive that nothing matches runs into its wait limit; a receive posted for another length than
    # the message reports the mismatch; messages of other pairs and later messages still work.
    code, err = run(bins, 2, "p2p_errors")
    assert code == 0, err


@needs2
def test_collective_next_to_compute(bins):
    # Allreduces on a side stream while a matmul loop keeps the compute stream busy (what
    # GradientBuckets.overlap_with_backward does): must finish well inside the wait limit.
    code, err = run(bins, min(NGPU, 4), "overlap", env={"IBCOMM_TIMEOUT_MS": "5000"})
    assert code == 0, err


@pytest.mark.skipif(NGPU < 3, reason="needs at least three GPUs")
def test_survivors_continue_on_gpus(bins):
    # After a rank has left between steps the others get the transport error, build a communicator over
    # the remaining ranks and carry on with device allreduces.  NVLS off (see test_rank_leaving_is_detected).
    code, err = run(bins, min(NGPU, 4), "leave_subset", env={"IBCOMM_DISABLE_NVLS": "1", "NCCL_NVLS_ENABLE": "0"})
    assert code == 0, err


@needs2
def test_chunk_size_on_real_gpus(bins):
    for chunk in (4, 32, 128):
        cmd = ["timeout", "120s", bins["ibcomm_run"], "-np", "2", "-x", f"IBCOMM_CHUNKSIZE={chunk}", bins["allreduce_tester"],
               "--device", "cuda", "ring", "1k", "i*np+p", "i*np*np+np*(np-1)/2"]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        assert p.returncode == 0, p.stderr[-2000:]


@needs2
@pytest.mark.slow
def test_aging_on_real_gpus(bins):
    np_ = min(NGPU, 4)
    for algo in ("ring", "rabenseifner"):
        cmd = ["timeout", "600s", bins["ibcomm_run"], "-np", str(np_), bins["allreduce_tester"], "--device", "cuda", "--iters", "100",
               algo, "128M", "i*np+p", "i*np*np+np*(np-1)/2"]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        assert p.returncode == 0, p.stderr[-2000:]
