"""CUDA kernels of the package and their Python face."""

from .build import KernelBuildError, compile_all, compile_library, load_library, source_names
from .kernels import KernelError
from .linear import linear, linear_into_stream, linear_norm, linear_silu

__all__ = ["KernelBuildError", "KernelError", "compile_all", "compile_library", "linear", "linear_into_stream", "linear_norm", "linear_silu",
           "load_library", "source_names"]
