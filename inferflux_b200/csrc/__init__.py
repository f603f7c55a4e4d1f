"""Hand-written CUDA kernels for sm_100a, their build and their Python table."""
from .build import BuildError, build, load_library
from .ops import CudaKernels, KernelError, PartialSum, ScaledRows

__all__ = ["BuildError", "build", "load_library", "CudaKernels", "KernelError", "PartialSum", "ScaledRows"]
