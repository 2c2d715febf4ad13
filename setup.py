"""Build hook: the sm_100a kernel library is compiled in-tree by nvcc before the Python files are collected, so
that wheels carry ``libcubic_b200.so`` with its bundle manifest.  All metadata lives in ``pyproject.toml``."""
import importlib.util
from pathlib import Path

from setuptools import setup
from setuptools.command.build_py import build_py


def _native():
    # loaded by path: importing the package would import torch, which a build environment need not have
    spec = importlib.util.spec_from_file_location("_cubic_native_build", Path(__file__).parent / "cubic_serve_b200" / "ops" / "native.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class BuildWithKernels(build_py):
    def run(self):
        native = _native()
        if native.needs_build():
            native.build()
        problems = native.verify_bundle()
        if problems:
            raise RuntimeError("native bundle does not match its sources: " + "; ".join(problems))
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
