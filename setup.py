"""Builds the native parts in-tree before packaging: the sm_100a kernel library (nvcc) and the transport daemon (g++).

The reference's ``setup.py`` downloads or builds the Go ``p2pd`` binary and compiles its protobuf files
(setup.py:82-162 there); here the daemon is a single C++ file, the protobuf classes are built at import time from
tables, and the CUDA kernels are compiled for ``compute_100a`` with ``nvcc``. Set ``HIVEMIND_B200_SKIP_NATIVE=1`` to
package without compiling (the library then builds itself on first use if ``nvcc`` is present).
"""
import os

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        if os.environ.get("HIVEMIND_B200_SKIP_NATIVE", "0") != "1":
            import importlib.util
            import pathlib

            spec = importlib.util.spec_from_file_location(
                "_hm_build", pathlib.Path(__file__).parent / "hivemind_b200" / "ops" / "_build.py")
            module = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(module)
            module.build_all()
        super().run()


setup(cmdclass={"build_py": BuildNative})
