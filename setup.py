"""Packaging of fastmoe_b200 (and the `fmoe` / `fmoe_cuda` import aliases).

The native extension targets sm_100a only (`-gencode arch=compute_100a,code=sm_100a`); the
reference's setup.py passes no architecture flag and relies on TORCH_CUDA_ARCH_LIST.  The
extension is compiled in-tree by `python -m fastmoe_b200.build` (run here as part of `build_py`
unless FMOE_SKIP_NATIVE_BUILD=1) and shipped as package data.
"""
import os

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py


class BuildWithNative(build_py):
    def run(self):
        if os.environ.get("FMOE_SKIP_NATIVE_BUILD", "0") != "1":
            from fastmoe_b200 import build as native_build
            native_build.build()
        super().run()


setup(
    name="fastmoe_b200",
    version="0.2.0",
    description="Mixture-of-Experts training system for NVIDIA B200 with the FastMoE API",
    packages=find_packages(include=["fastmoe_b200", "fastmoe_b200.*", "fmoe"]),
    py_modules=["fmoe_cuda"],
    package_data={"fastmoe_b200": ["_build/*.so", "csrc/*", "csrc/*/*"]},
    install_requires=["torch", "numpy"],
    cmdclass={"build_py": BuildWithNative},
)
