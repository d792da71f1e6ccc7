# SPDX-License-Identifier: MIT
"""In-tree build of the `_C` extension for sm_100a.

The reference builds one CUDAExtension from core.cu, binding.cpp and w8a16.cu
with the arch taken from TORCH_CUDA_ARCH_LIST (torch_ext/setup.py:21-41).
Here the arch is fixed: every kernel is written for sm_100a (tcgen05, TMA,
multimem), so the build passes its own -gencode and nothing else.

The product of a build is `_build/_C.so` next to this file.  It is loaded by
`barlink_sm86_b200/__init__.py`; nothing is installed into site-packages.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD_DIR = os.path.join(HERE, "_build")

SOURCES = [
    "heap.cc",
    "comm_kernels.cu",
    "gemm_kernels.cu",
    "dlin_kernels.cu",
    "ops_kernels.cu",
    "attn_kernels.cu",
    "attn_tc_kernels.cu",
    "w8a16_kernels.cu",
    "w4a16_kernels.cu",
    "backend.cc",
    "binding.cc",
    "binding_extra.cc",
]

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-Wno-unused-function"]


def so_path():
    return os.path.join(BUILD_DIR, "_C.so")


def build(verbose=False):
    """Compile (or incrementally rebuild) the extension; returns the module."""
    if "barlink_sm86_b200._C" in sys.modules:
        # already loaded in this process: rebuild in a child (importing the shared object a second
        # time would register its classes twice); the running process keeps the module it has
        import subprocess

        subprocess.check_call([sys.executable, os.path.abspath(__file__)] + (["-v"] if verbose else []))
        return sys.modules["barlink_sm86_b200._C"]
    from torch.utils import cpp_extension

    os.makedirs(BUILD_DIR, exist_ok=True)
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    jobs = os.environ.get("MAX_JOBS")
    if jobs is None:
        os.environ["MAX_JOBS"] = str(max(1, (os.cpu_count() or 2)))
    mod = cpp_extension.load(
        name="_C",
        sources=srcs,
        extra_cflags=CXX_FLAGS,
        extra_cuda_cflags=NVCC_FLAGS,
        extra_include_paths=[CSRC],
        build_directory=BUILD_DIR,
        with_cuda=True,
        verbose=verbose,
    )
    # the build imports the module; the package must use this instance (loading the
    # same shared object a second time would register its classes twice)
    sys.modules["barlink_sm86_b200._C"] = mod
    return mod


if __name__ == "__main__":
    build(verbose="-v" in sys.argv)
    print(so_path())
