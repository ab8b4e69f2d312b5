"""Host transport and schedule simulator: the C++ binaries `sendrecv`
(loop-back endpoints in one process, like the reference's
tests/sendrecv_test.cpp) and `schedule_sim` (every device op program
interpreted on CPU threads for world sizes 2..8)."""
import subprocess


def test_sendrecv_binary(bins):
    p = subprocess.run([bins["sendrecv"]], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert p.returncode == 0, p.stdout


def test_schedule_simulator(bins):
    p = subprocess.run([bins["schedule_sim"]], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert p.returncode == 0, p.stdout
