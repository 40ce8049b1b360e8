"""CUDA kernels for sm_100a: build (nvcc, in-tree), loading (ctypes) and their Python faces."""
from .build import KernelBuildError, build_all, library

__all__ = ["KernelBuildError", "build_all", "library"]
