"""Build script: compiles the sm_100a extension in place.

    python setup.py build_ext --inplace

The extension targets Blackwell only (``-gencode arch=compute_100a,code=sm_100a``);
passing the arch flags explicitly bypasses torch's own architecture list, so the
build also works on a machine without a GPU.
"""

import glob
import os

from setuptools import find_packages, setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join('megablocks_b200', 'csrc')

NVCC_FLAGS = [
    '-O3',
    '-std=c++17',
    '-gencode', 'arch=compute_100a,code=sm_100a',
    '-lineinfo',
    '--use_fast_math',
    '-Xptxas', '-v',
    '--expt-relaxed-constexpr',
    '-U__CUDA_NO_HALF_OPERATORS__',
    '-U__CUDA_NO_HALF_CONVERSIONS__',
    '-U__CUDA_NO_BFLOAT16_CONVERSIONS__',
]

# MB200_GEMM_TIMING=1: diagnostic build whose grouped GEMM records per-role wait cycles
# (read back with `_C.gemm_role_timers`).
DEFINES = ['-DMB_GEMM_TIMING'] if os.environ.get('MB200_GEMM_TIMING') == '1' else []
if os.environ.get('MB200_GEMM_NO_STORE') == '1':   # diagnostic: epilogue without its global stores
    DEFINES.append('-DMB_GEMM_NO_STORE')
NVCC_FLAGS += DEFINES

sources = sorted(glob.glob(os.path.join(CSRC, '*.cu'))) + sorted(glob.glob(os.path.join(CSRC, '*.cpp')))

setup(
    name='megablocks_b200',
    version='0.1.0',
    packages=find_packages(exclude=('tests', 'baseline', 'profiles')),
    ext_modules=[
        CUDAExtension(
            name='megablocks_b200._C',
            sources=sources,
            include_dirs=[os.path.join(ROOT, CSRC)],
            extra_compile_args={'cxx': ['-O3', '-std=c++17'] + DEFINES, 'nvcc': NVCC_FLAGS},
        )
    ],
    cmdclass={'build_ext': BuildExtension.with_options(use_ninja=True)},
)
