from . import build, kernels
from .kernels import KernelError

__all__ = ["build", "kernels", "KernelError"]
