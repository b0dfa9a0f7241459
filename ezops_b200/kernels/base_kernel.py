"""Abstract kernel: one callable object per (op, backend) (ezops/kernels/base_kernel.py:4-6)."""

from abc import ABC, abstractmethod


class BaseKernel(ABC):
    @abstractmethod
    def __call__(self, *args, **kwargs): ...
