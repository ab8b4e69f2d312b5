"""Packaging shim: `pip install .` (or `python setup.py build`) first runs the
in-tree build (explicit nvcc / g++ command lines for sm_100a, see
allreduce_proto_b200/build.py), so that the shared library is there to be
packaged.  The library is loaded from `allreduce_proto_b200/_lib/`; when it is
missing at import time the package builds it on first use."""
import importlib.util
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNativeFirst(build_py):
    def run(self):
        spec = importlib.util.spec_from_file_location("_ibcomm_build", Path(__file__).parent / "allreduce_proto_b200" / "build.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
        super().run()


setup(cmdclass={"build_py": BuildNativeFirst})
