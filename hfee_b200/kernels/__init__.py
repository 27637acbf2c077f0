from . import build, ops
from .ops import KernelLibraryError

__all__ = ["build", "ops", "KernelLibraryError"]
