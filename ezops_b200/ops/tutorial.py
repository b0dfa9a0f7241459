"""The reference's three small teaching operators, kept for API completeness:
``VectorAddOp`` (ezops/ops/vector_add.py:7-30), ``SoftmaxOp``
(ezops/ops/softmax.py:7-36) and ``ReduceOp`` (ezops/ops/reduce.py:7-33).  Same
constructors, ``forward`` signatures (results written into the last argument),
workloads and tolerances; ``gen_data`` additionally takes ``device``.
"""

from __future__ import annotations

import torch

from ..registry import get_kernel
from .base_op import Op


class VectorAddOp(Op):
    _params_desc = {"n": "Number of elements"}

    def __init__(self, n: int, backend: str = "ref"):
        self.n, self._backend = n, backend
        self._kernel = self._ref_forward if backend == "ref" else get_kernel("vector_add", backend)(n=n)

    def forward(self, A, B, C) -> None:
        self._kernel(A, B, C)

    def gen_data(self, device="cuda"):
        kw = dict(device=device, dtype=torch.float32)
        return torch.randn(self.n, **kw), torch.randn(self.n, **kw), torch.empty(self.n, **kw)

    def _ref_forward(self, A, B, C) -> None:
        C.copy_(A + B)


class SoftmaxOp(Op):
    _params_desc = {"batch_size": "Number of rows", "dim": "Feature dimension per row (softmax over dim)"}
    _atol = 1e-6
    _rtol = 1e-5

    def __init__(self, batch_size: int, dim: int, backend: str = "ref"):
        self.batch_size, self.dim, self._backend = batch_size, dim, backend
        self._kernel = self._ref_forward if backend == "ref" else get_kernel("softmax", backend)(batch_size=batch_size, dim=dim)

    def forward(self, X, Out) -> None:
        self._kernel(X, Out)

    def gen_data(self, device="cuda"):
        kw = dict(device=device, dtype=torch.float32)
        return torch.randn(self.batch_size, self.dim, **kw), torch.empty(self.batch_size, self.dim, **kw)

    def _ref_forward(self, X, Out) -> None:
        Out.copy_(torch.softmax(X, dim=-1))


class ReduceOp(Op):
    _params_desc = {"n": "Number of input elements"}

    def __init__(self, n: int, backend: str = "ref"):
        self.n, self._backend = n, backend
        # summation order differs between implementations and the error grows with n
        self._atol = 1e-7 * n
        self._kernel = self._ref_forward if backend == "ref" else get_kernel("reduce", backend)(n=n)

    def forward(self, A, Out) -> None:
        self._kernel(A, Out)

    def gen_data(self, device="cuda"):
        return torch.randn(self.n, device=device, dtype=torch.float32), torch.empty(1, device=device, dtype=torch.float32)

    def _ref_forward(self, A, Out) -> None:
        Out.copy_(A.sum())
