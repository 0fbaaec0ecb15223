"""Bindings of the CUDA library built from ``csrc`` and the choice of matrix product."""

from .build import BuildError, build_library, library
from .kernels import KernelError
from .linear import linear

__all__ = ["BuildError", "KernelError", "build_library", "library", "linear"]
