from .api import CudaKernels, KernelError, KernelSet
from .build import BuildError, build_all

__all__ = ["CudaKernels", "KernelError", "KernelSet", "BuildError", "build_all"]
