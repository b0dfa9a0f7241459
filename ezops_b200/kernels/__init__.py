"""Kernel backends.  Importing this package registers the sm_100a kernels; it
raises if ``libezb200.so`` has not been built (there is no fallback)."""

from . import sm100  # noqa: F401
from .base_kernel import BaseKernel

__all__ = ["BaseKernel"]
