"""Packaging: ``pip install -e .`` builds the sm_100a kernel library in-tree and installs ``teletron_b200``."""

import os
import subprocess
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py


class BuildWithKernels(build_py):
    def run(self):
        here = os.path.dirname(os.path.abspath(__file__))
        subprocess.check_call([sys.executable, "-m", "teletron_b200.build"], cwd=here)
        super().run()


setup(
    name="teletron_b200",
    version="0.1.0",
    description="Blackwell-native long-context video-DiT training framework with TeleTron's capabilities",
    packages=find_packages(include=["teletron_b200", "teletron_b200.*"]),
    package_data={"teletron_b200": ["lib/*.so", "csrc/*", "data/*.yml", "convert_ckpt/hunyuan/*.sh", "convert_ckpt/hunyuan/*.md"]},
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "numpy", "pyyaml", "transformers"],
    cmdclass={"build_py": BuildWithKernels},
)
