"""The hand-written CUDA kernels: building them (``build``) and calling them (``ops``)."""

from . import ops
from .build import BuildError, build_library
from .ops import KernelError

__all__ = ["BuildError", "KernelError", "build_library", "ops"]
