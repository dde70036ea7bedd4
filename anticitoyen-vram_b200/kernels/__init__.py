"""Hand-written CUDA kernels for sm_100a and their Python faces.

``ops`` holds one function per kernel; ``build`` compiles ``csrc/`` on first use.
"""

from . import ops
from .build import BuildError, library_path
from .ops import KernelError

__all__ = ["BuildError", "KernelError", "library_path", "ops"]
