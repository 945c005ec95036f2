"""CUDA kernels for sm_100a and their Python entry points.

`ops` holds one checked entry point per kernel; `reference` holds a plain PyTorch
statement of each kernel's arithmetic, used by the tests and nowhere on the product
path.  `require_kernels()` is called when an engine is built so that a missing
compiler or library stops start-up rather than the first step.
"""

from .library import KernelError, library, library_path


def require_kernels() -> str:
    """Build (if needed) and load the CUDA library; return its path.  Raises KernelError."""
    library()
    return library_path()


__all__ = ["KernelError", "library", "library_path", "require_kernels"]
