"""Compiles the sm_100a kernels into ``nanopysche_b200/lib/libnpb200.so`` (when nvcc is available) as part of the
build; without a toolchain the library is built on first use on a machine that has one."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class build_py_with_kernels(build_py):
    def run(self):
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        try:
            from nanopysche_b200.build import build_extension

            print("built", build_extension())
        except Exception as e:  # noqa: BLE001
            print(f"nanopysche_b200: kernels not built ({e})")
        super().run()


setup(cmdclass={"build_py": build_py_with_kernels})
