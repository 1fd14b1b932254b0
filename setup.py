"""Builds libleapquant_b200.so with nvcc (sm_100a) before the Python files are collected, so that `pip install .` ships the
library inside the package.  All project metadata lives in pyproject.toml."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


class BuildWithLibrary(build_py):
    def run(self):
        from leapquant_b200.csrc import build as native
        native.build()
        super().run()


setup(cmdclass={"build_py": BuildWithLibrary})
