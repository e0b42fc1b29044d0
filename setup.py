"""Builds ``offload_adam_b200._C`` for sm_100a with the same flags as the in-tree
build (``offload_adam_b200/_ext.py``).  ``pip install --no-build-isolation -e .`` or
``python setup.py build_ext --inplace``; nvcc is required, a GPU is not."""

import glob
import os

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join("offload_adam_b200", "csrc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--fmad=false",
    "--expt-relaxed-constexpr", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
]

os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")  # only consulted for its presence; -gencode above decides

setup(
    ext_modules=[
        CUDAExtension(
            name="offload_adam_b200._C",
            sources=sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp"))),
            include_dirs=[os.path.join(HERE, CSRC)],
            extra_compile_args={"cxx": ["-O3", "-std=c++17"], "nvcc": NVCC_FLAGS},
        )
    ],
    cmdclass={"build_ext": BuildExtension.with_options(use_ninja=True)},
)
