"""Build entry of the `custom_modules` torch extension (drop-in for the
reference's setup.py, which builds the same module name from modules.cpp and
cuda/dit.cu).

    python sd3.c_b200/setup.py build_ext --inplace

First builds libsd3_b200.so (CUDA kernels + C ABI, nvcc, sm_100a) through
build.py, then compiles modules.cpp against torch and links it to that
library with an $ORIGIN rpath, so both files sit side by side in this
directory.
"""
import os
import sys

from setuptools import setup
from torch.utils.cpp_extension import BuildExtension, CppExtension

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import build as sd3_build  # noqa: E402

sd3_build.build()
os.chdir(HERE)

setup(
    name="custom_modules",
    ext_modules=[
        CppExtension(
            "custom_modules",
            ["modules.cpp"],
            include_dirs=[os.path.join(HERE, "..", "include"), "/usr/local/cuda/include"],
            library_dirs=[HERE, "/usr/local/cuda/lib64"],
            libraries=["sd3_b200", "cudart", "c10_cuda", "torch_cuda"],
            extra_compile_args=["-O2", "-std=c++17"],
            extra_link_args=["-Wl,-rpath,$ORIGIN"],
        ),
    ],
    cmdclass={"build_ext": BuildExtension.with_options(no_python_abi_suffix=True)},
)
