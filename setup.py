"""Packaging: builds the native library in-tree with `make` (nvcc for sm_100a, system g++) and ships it inside the wheel.

    pip install --no-build-isolation .        # or: python setup.py bdist_wheel

The reference drives cmake from its setup.py the same way (src/smem/python/memfabric_hybrid/setup.py)."""
import os
import subprocess

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildNative(build_py):
    def run(self):
        subprocess.check_call(["make", "-j", str(os.cpu_count() or 8)], cwd=ROOT)
        super().run()


setup(
    name="memfabric_hybrid_b200",
    version="1.0.0",
    description="Blackwell-native memory fabric: pooled HBM/DRAM over a global virtual address space, xcopy, fused collectives",
    packages=find_packages(include=["memfabric_hybrid_b200", "memfabric_hybrid_b200.*", "memfabric_hybrid", "mf_adapter"]),
    package_data={"memfabric_hybrid_b200": ["lib/*.so", "*.so"]},
    include_package_data=True,
    cmdclass={"build_py": BuildNative},
    python_requires=">=3.10",
)
