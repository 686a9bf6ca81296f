"""``pip install -e .`` for the framework: builds the in-tree CUDA extension (sm_100a) with ``build_ext.py``
and installs the ``kolmogorov_moe_architecture_b200`` package plus the ``moe_arch`` import shim."""
import os
import subprocess
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildWithKernels(build_py):
    def run(self):
        if os.environ.get("KMOE_SKIP_KERNEL_BUILD", "0") != "1":
            subprocess.check_call([sys.executable, os.path.join(ROOT, "build_ext.py")])
        super().run()


setup(
    name="kolmogorov_moe_architecture_b200",
    version="0.1.0",
    description="B200-native hybrid MoE training framework (API of Kolmogorov-MoE-Architecture)",
    packages=find_packages(include=["kolmogorov_moe_architecture_b200*", "moe_arch*"]),
    package_data={"kolmogorov_moe_architecture_b200": ["_C.so", "csrc/*"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "numpy", "pyyaml"],
    cmdclass={"build_py": BuildWithKernels},
)
