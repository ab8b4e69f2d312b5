"""Multi-process tests on CPU: the Python Communicator over the shared-memory
host transport (world sizes 2-5), two-sided messaging, broadcast, and failure
detection without a GPU (a rank that exits, a rank that never joins, a rank
killed in the middle of a collective)."""
import os
import signal
import subprocess
import sys
import time
from pathlib import Path

import pytest

WORKER = str(Path(__file__).resolve().parent / "host_worker.py")


def run(bins, np, case, env=None, timeout=180):
    cmd = ["timeout", f"{timeout}s", bins["ibcomm_run"], "-np", str(np)]
    for k, v in (env or {}).items():
        cmd += ["-x", f"{k}={v}"]
    cmd += [sys.executable, WORKER, case]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    return p.returncode, p.stderr[-3000:]


@pytest.mark.parametrize("np_", [2, 4])
def test_allreduce_4mi_fp32_against_serial_sum(bins, np_):
    code, err = run(bins, np_, "allreduce")
    assert code == 0, err


@pytest.mark.parametrize("np_", [3, 5])
def test_allreduce_non_power_of_two(bins, np_):
    code, err = run(bins, np_, "allreduce")
    assert code == 0, err


@pytest.mark.parametrize("np_", [1, 2, 5, 8])
def test_ranks_as_threads_of_one_process(bins, np_):
    # The second process model: N host threads, one communicator each.
    p = subprocess.run(["timeout", "120s", bins["threads_test"], "cpu", str(np_)], stdout=subprocess.PIPE,
                       stderr=subprocess.PIPE, text=True)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "threads_test OK" in p.stdout


@pytest.mark.parametrize("np_", [2, 3, 5])
def test_reduce_scatter_and_all_gather_on_host_buffers(bins, np_):
    code, err = run(bins, np_, "rsag")
    assert code == 0, err


def test_sharded_gradient_buckets_on_host_tensors(bins):
    code, err = run(bins, 3, "sharded_buckets")
    assert code == 0, err


def test_messaging_and_bcast(bins):
    code, err = run(bins, 3, "messaging")
    assert code == 0, err


def test_peer_that_exits_is_detected(bins):
    t0 = time.time()
    code, err = run(bins, 3, "peer_exit", env={"IBCOMM_RUN_GRACE_MS": "20000"})
    assert code == 0, err
    assert time.time() - t0 < 60


def test_survivors_form_a_smaller_communicator(bins):
    # Elastic shrink on the host: a rank leaves between steps, the others get the transport
    # error, build a communicator over the survivors and finish the work.
    code, err = run(bins, 4, "shrink", env={"IBCOMM_RUN_GRACE_MS": "30000"})
    assert code == 0, err


def test_rank_that_never_joins(bins, tmp_path):
    """Bootstrap gives up with the transport error code when a rank is missing."""
    env = dict(os.environ, IBCOMM_RANK="0", IBCOMM_WORLD_SIZE="2", IBCOMM_BOOTSTRAP_DIR=str(tmp_path))
    code = subprocess.run([sys.executable, "-c", (
        "import sys; sys.path.insert(0, %r)\n"
        "import allreduce_proto_b200 as ar\n"
        "try:\n"
        "    ar.Communicator.from_env(timeout_s=1.0)\n"
        "except ar.IbcommError as e:\n"
        "    sys.exit(e.code)\n"
        "sys.exit(0)\n") % str(Path(WORKER).parent.parent)], env=env).returncode
    assert code == 2


def test_rank_killed_mid_collective_fails_the_others(bins):
    """A tester rank is killed while a long allreduce runs; the launcher must
    return non-zero well before the shell timeout, and the survivors exit with
    the transport error code (2) rather than spinning forever."""
    cmd = ["timeout", "120s", bins["ibcomm_run"], "-np", "3", "-x", "IBCOMM_TIMEOUT_MS=2000", bins["allreduce_tester"],
           "--device", "cpu", "--iters", "400", "ring", "64M", "1", "np"]
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    time.sleep(2.0)
    # kill one rank (a child of the launcher) by its exact pid
    kids = subprocess.run(["ps", "-o", "pid=", "--ppid", str(p.pid)], stdout=subprocess.PIPE, text=True).stdout.split()
    launcher_kids = []
    for k in kids:
        launcher_kids += subprocess.run(["ps", "-o", "pid=", "--ppid", k], stdout=subprocess.PIPE, text=True).stdout.split()
    victims = launcher_kids or kids
    assert victims, "no rank processes found"
    os.kill(int(victims[-1]), signal.SIGKILL)
    t0 = time.time()
    out, err = p.communicate(timeout=100)
    assert p.returncode != 0
    assert time.time() - t0 < 60
    assert p.returncode in (2, 137), (p.returncode, err[-2000:])


def test_trace_file_format(bins, tmp_path):
    prefix = str(tmp_path / "tr")
    code, err = run(bins, 2, "trace", env={"IBCOMM_TRACE": "1", "IBCOMM_TRACE_FILE": prefix})
    assert code == 0, err
    for r in range(2):
        lines = Path(f"{prefix}_{r}.dat").read_text().splitlines()
        names = [ln.split(",")[0] for ln in lines]
        assert names == ["received", "reduced", "issue_send", "issue_copy_kernel", "issue_redu_kernel", "issue_recv", "other"]


@pytest.mark.parametrize("sharded", [False, True, "overlap"])
def test_data_parallel_example_on_cpu(sharded):
    # examples/ddp_gradient_buckets.py under torchrun (gloo only for the rendezvous store): real autograd
    # gradients in buckets, averaged over the library's host transport; the ranks must end with equal weights.
    example = str(Path(__file__).resolve().parent.parent / "examples" / "ddp_gradient_buckets.py")
    port = 29650 + [False, True, "overlap"].index(sharded)
    cmd = ["timeout", "300s", sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "3",
           "--master-addr", "127.0.0.1", "--master-port", str(port), example, "--device", "cpu", "--steps", "3"]
    if sharded == "overlap":
        cmd.append("--overlap")
    elif sharded:
        cmd.append("--sharded")
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert p.returncode == 0, p.stdout[-3000:]
    assert p.stdout.count(": OK") == 3, p.stdout[-3000:]
