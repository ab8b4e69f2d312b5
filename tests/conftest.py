"""Test configuration: markers, one in-tree build per session, helper paths."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a GPU machine)")
    config.addinivalue_line("markers", "slow: long-running soak tests")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


@pytest.fixture(scope="session", autouse=True)
def built():
    """Builds the native library and the tools once (no-op when up to date)."""
    from allreduce_proto_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def bins(built):
    return {k: str(v) for k, v in built.items() if v is not None}


def run_ranks(bins, np, args, env=None, timeout=120):
    """`timeout Ns ibcomm_run -np N [-x K=V] program args...` -> exit status."""
    cmd = ["timeout", f"{timeout}s", bins["ibcomm_run"], "-np", str(np)]
    for k, v in (env or {}).items():
        cmd += ["-x", f"{k}={v}"]
    cmd += list(args)
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    return p.returncode, p.stdout, p.stderr


@pytest.fixture(scope="session")
def ranks(bins):
    def _run(np, args, env=None, timeout=120):
        return run_ranks(bins, np, args, env, timeout)
    return _run
