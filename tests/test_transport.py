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


def test_schedule_simulator_under_thread_sanitizer(tmp_path):
    """The flag protocol of the op programs (release store of a flag after the
    data, acquire load before reading it, credits before a slot is reused) is
    replayed on CPU threads under ThreadSanitizer: any data race between the
    emulated ranks or channels is reported."""
    import shutil
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    if shutil.which("g++") is None:
        import pytest
        pytest.skip("no g++")
    exe = tmp_path / "schedule_sim_tsan"
    srcs = ["tests/cpp/schedule_sim.cpp"] + [f"src/host/{n}.cpp" for n in
            ("error", "env", "partition", "schedule", "tunables", "shm_transport", "trace", "communicator")]
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-w", f"-I{root / 'include'}", f"-I{root / 'tests' / 'cpp'}",
           *[str(root / s) for s in srcs], "-o", str(exe), "-pthread", "-lrt"]
    b = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if b.returncode != 0 and "tsan" in b.stdout.lower():
        import pytest
        pytest.skip("ThreadSanitizer runtime not available")
    assert b.returncode == 0, b.stdout[-2000:]
    p = subprocess.run([str(exe)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
    assert p.returncode == 0, p.stdout[-3000:]
    assert "ThreadSanitizer" not in p.stdout, p.stdout[-3000:]


def test_two_shot_window_protocol(bins):
    # The staged two-shot allreduce and reduce-scatter / all-gather protocols
    # (per-CTA barriers, the same split of every window) as CPU threads.
    p = subprocess.run([bins["twoshot_sim"]], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert p.returncode == 0, p.stdout


def test_two_shot_window_protocol_under_thread_sanitizer(tmp_path):
    """A CTA that could run ahead into bytes another CTA has not copied out yet is
    a data race between the threads of this model; ThreadSanitizer reports it."""
    import shutil
    from pathlib import Path
    import pytest
    root = Path(__file__).resolve().parent.parent
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = tmp_path / "twoshot_sim_tsan"
    srcs = ["tests/cpp/twoshot_sim.cpp"] + [f"src/host/{n}.cpp" for n in
            ("error", "env", "partition", "schedule", "tunables", "shm_transport", "trace", "communicator")]
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-w", f"-I{root / 'include'}", f"-I{root / 'tests' / 'cpp'}",
           *[str(root / s) for s in srcs], "-o", str(exe), "-pthread", "-lrt"]
    b = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if b.returncode != 0 and "tsan" in b.stdout.lower():
        pytest.skip("ThreadSanitizer runtime not available")
    assert b.returncode == 0, b.stdout[-2000:]
    p = subprocess.run([str(exe)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=900)
    assert p.returncode == 0, p.stdout[-3000:]
    assert "ThreadSanitizer" not in p.stdout, p.stdout[-3000:]
