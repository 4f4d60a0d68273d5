"""Packaging shim: ``pip install -e .`` (or ``python setup.py build_py``) compiles the CUDA kernels for
sm_100a and the host C++ in-tree with ``zenyx_b200/_build.py`` (nvcc and g++ must be on the machine; no
GPU is needed to build) and ships the two shared objects as package data."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


class BuildWithKernels(build_py):
    def run(self):
        from zenyx_b200 import _build

        _build.build_all(verbose=False)
        super().run()


setup(cmdclass={"build_py": BuildWithKernels})
