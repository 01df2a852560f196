"""Build of the B200 kernel library and its torch binding.

Takes the place of the reference's setup.py (:23-51), which compiles src/rmsnorm_kernel.cu and
pytorch_binding/binding.cpp into one CUDAExtension for whatever architectures torch lists. Here:

  1. `mgrrmsnorm_b200/build.py` compiles every kernel source with nvcc for ONE architecture
     (-gencode arch=compute_100a,code=sm_100a) into the C-ABI library mgrrmsnorm_b200/lib/libmgr_b200.so;
  2. pytorch_binding/binding.cpp (plain C++, no kernels) becomes the torch extension `rmsnorm_cuda_ops`,
     placed in mgrrmsnorm_b200/pybind/ and linked against that library.

No Triton requirement, no multi-architecture fat binary, no `--use_fast_math`, no CPU fallback.

    python setup.py build_ext --inplace        # or: pip install --no-build-isolation -e .
"""
import os
import sys
from pathlib import Path

from setuptools import find_packages, setup
from torch.utils.cpp_extension import BuildExtension, CUDAExtension

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
from mgrrmsnorm_b200 import build as kernel_build  # noqa: E402  (no torch, no CUDA needed to import)


class BuildKernelsThenBinding(BuildExtension):
    """Builds libmgr_b200.so first (the binding links against it), then the extension."""

    def run(self):
        kernel_build.build()
        super().run()


setup(
    name="mgrrmsnorm_b200",
    version="0.1.0",
    description="B200 (sm_100a) RMSNorm and SwiGLU MLP kernels behind the megagemm operator API",
    packages=find_packages(include=["mgrrmsnorm_b200", "mgrrmsnorm_b200.*", "megagemm"]),
    py_modules=["rmsnorm_cuda_ops"],
    package_data={"mgrrmsnorm_b200": ["lib/libmgr_b200.so"]},
    ext_modules=[
        CUDAExtension(
            name="mgrrmsnorm_b200.pybind.rmsnorm_cuda_ops",
            sources=["pytorch_binding/binding.cpp"],          # host code only: the kernels are in the library
            include_dirs=[str(ROOT / "include")],
            library_dirs=[str(ROOT / "mgrrmsnorm_b200" / "lib")],
            libraries=["mgr_b200"],
            extra_compile_args={"cxx": ["-O2", "-std=c++17"]},
            extra_link_args=["-Wl,-rpath,$ORIGIN/../lib"],    # finds the library next to the package, wherever it is installed
        ),
    ],
    cmdclass={"build_ext": BuildKernelsThenBinding.with_options(use_ninja=bool(int(os.environ.get("MGR_USE_NINJA", "1"))))},
    install_requires=["torch>=2.0"],
    python_requires=">=3.9",
)
