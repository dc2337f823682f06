"""Packaging entry point.  ``pip install .`` (or ``-e .``) compiles the sm_100a kernels with
nvcc into ``elf_b200/csrc/_build`` before the Python files are collected, so the wheel ships
the extension next to its sources.  ``ELF_B200_SKIP_BUILD=1`` skips the compilation (the
kernels can be built later with ``python -m elf_b200.csrc.build``); without nvcc the build is
skipped with a warning and the package runs on CPU / torch fallbacks only."""

import os
import shutil
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class build_py_with_kernels(build_py):
    def run(self):
        if os.environ.get("ELF_B200_SKIP_BUILD", "0") == "1":
            print("ELF_B200_SKIP_BUILD=1: not compiling the CUDA extension", file=sys.stderr)
        elif shutil.which("nvcc") is None:
            print("warning: nvcc not found, the CUDA extension is not built", file=sys.stderr)
        else:
            here = os.path.dirname(os.path.abspath(__file__))
            sys.path.insert(0, here)
            try:
                from elf_b200.csrc.build import build

                build(verbose=False)
            finally:
                sys.path.remove(here)
        super().run()


setup(cmdclass={"build_py": build_py_with_kernels})
