"""Builds the package's sm_100a kernels (when nvcc is available) before the files are collected; the pure-PyTorch
paths work without them, so a missing toolchain is not an error."""
import os
import sys

from setuptools import setup
from setuptools.command.build_py import build_py


class build_py_with_kernels(build_py):
    def run(self):
        here = os.path.dirname(os.path.abspath(__file__))
        sys.path.insert(0, os.path.dirname(here))
        try:
            import importlib.util

            spec = importlib.util.spec_from_file_location("_fp8_flow_moe_build", os.path.join(here, "build.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            print("built", mod.build_extension())
        except Exception as e:  # noqa: BLE001
            print(f"fp8_flow_moe: kernels not built ({e}); they are built on first use if nvcc shows up")
        super().run()


setup(cmdclass={"build_py": build_py_with_kernels})
