"""The reference's small teaching operators, kept for API completeness:
``VectorAddOp`` (ezops/ops/vector_add.py:7-30), ``SoftmaxOp``
(ezops/ops/softmax.py:7-36), ``ReduceOp`` (ezops/ops/reduce.py:7-33) and
``PdlGemmOp`` (ezops/ops/pdl_gemm.py:7-76).  Same
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


class PdlGemmOp(Op):
    """Two chained GEMMs, y = x @ W1 and z = y @ W2 (fp32 tensors), the workload on which the reference shows
    programmatic dependent launch (ezops/ops/pdl_gemm.py:7-76).  Backends: ``"ref"`` (torch), ``"cuda"`` (two ordinary
    launches) and ``"cuda_pdl"`` (the second launch may start while the first drains)."""

    _params_desc = {
        "M": "Batch / sequence dimension (rows of x, y, z)",
        "K": "Input feature dimension (cols of x, rows of W1)",
        "N": "Hidden dimension (cols of W1, rows of W2)",
        "P": "Output feature dimension (cols of W2)",
    }
    _atol = 1e-2
    _rtol = 1e-2

    def __init__(self, M: int, K: int, N: int, P: int, backend: str = "ref"):
        self.M, self.K, self.N, self.P, self._backend = M, K, N, P, backend
        self._kernel = self._ref_forward if backend == "ref" else get_kernel("pdl_gemm", backend)(M=M, K=K, N=N, P=P)

    def check(self, actual, expected) -> bool:
        """Relative Frobenius error below rtol: tensor-core backends round the inputs (TF32 here), which leaves an
        error floor relative to the largest outputs, not to each element (ezops/ops/pdl_gemm.py:21-37)."""
        if actual.shape != expected.shape:
            return False
        diff = (actual.float() - expected.float()).norm().item()
        return diff / max(expected.float().norm().item(), 1.0) < self._rtol

    def forward(self, x, W1, W2, y, z) -> None:
        self._kernel(x, W1, W2, y, z)

    def gen_data(self, device="cuda"):
        kw = dict(device=device, dtype=torch.float32)
        return (torch.randn(self.M, self.K, **kw), torch.randn(self.K, self.N, **kw), torch.randn(self.N, self.P, **kw),
                torch.empty(self.M, self.N, **kw), torch.empty(self.M, self.P, **kw))

    def _ref_forward(self, x, W1, W2, y, z) -> None:
        torch.matmul(x, W1, out=y)
        torch.matmul(y, W2, out=z)
