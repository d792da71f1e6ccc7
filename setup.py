# SPDX-License-Identifier: MIT
"""Packaging for users who want `pip install .` (the reference ships
torch_ext/setup.py:21-41 for the same purpose).  The extension is compiled for
sm_100a by `barlink_sm86_b200/_build.py` -- the arch is fixed, not taken from
TORCH_CUDA_ARCH_LIST, because every kernel is written for sm_100a -- and the
resulting `_build/_C.so` travels inside the package.  Development and the
tests use the tree in place (`python -m barlink_sm86_b200._build`)."""
import os
import sys

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


class BuildWithExtension(build_py):
    def run(self):
        if os.environ.get("BL_SKIP_EXT_BUILD") != "1":
            sys.path.insert(0, ROOT)
            from barlink_sm86_b200 import _build

            _build.build(verbose=False)
        super().run()


setup(
    name="barlink-b200",
    version="0.1.0",
    description="Blackwell-native peer-to-peer collectives and tensor-parallel inference kernels (barlink API)",
    packages=find_packages(include=["barlink_sm86_b200*", "barlink_sm86*", "vllm_barlink*"]),
    package_data={"barlink_sm86_b200": ["_build/_C*.so", "csrc/*"], "vllm_barlink": ["*.sh"]},
    python_requires=">=3.10",
    install_requires=["torch"],
    cmdclass={"build_py": BuildWithExtension},
)
