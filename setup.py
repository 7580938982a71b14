"""Packaging of kernel_b200.

    python setup.py build_ext --inplace     # nvcc build of kernel_b200/lib/libkb200.so (sm_100a; no GPU needed)
    pip install --no-build-isolation -e .   # the same, then a development install

The native library is not a Python extension module: it has a plain C ABI and is
loaded with ctypes, so ``build_ext`` only drives ``kernel_b200.csrc.build``.
"""
import sys
from pathlib import Path

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def _build_native(force: bool = False) -> None:
    from kernel_b200.csrc.build import build

    print(f"built {build(force=force)}")


class BuildNative(Command):
    description = "compile libkb200.so with nvcc for sm_100a"
    user_options = [("inplace", "i", "accepted for compatibility; the library is always built in-tree"),
                    ("force", "f", "rebuild even if the sources are unchanged")]
    boolean_options = ["inplace", "force"]

    def initialize_options(self):
        self.inplace = False
        self.force = False

    def finalize_options(self):
        pass

    def run(self):
        _build_native(bool(self.force))


class BuildPyWithNative(build_py):
    def run(self):
        _build_native()
        super().run()


setup(
    name="kernel_b200",
    version="0.1.0",
    description="Blackwell-native fused communication kernels (MoE all-to-all, GEMM+reduce-scatter, all-gather+GEMM) and their harness",
    packages=find_packages(include=["kernel_b200", "kernel_b200.*"]),
    package_data={"kernel_b200": ["lib/*.so", "csrc/**/*", "tasks/*/task.yml"]},
    python_requires=">=3.10",
    install_requires=["torch", "pyyaml"],
    cmdclass={"build_ext": BuildNative, "build_py": BuildPyWithNative},
)
