"""GEMV operator spec: C[N] = A[K] . B, bf16 in, fp32 accumulate, bf16 out
(ezops/ops/gemv.py:7-38).

Layout follows the reference: kernels receive B as [N, K] row-major (each
output element is one contiguous weight row); the torch ``"ref"`` backend
receives B as [K, N] and computes ``A @ B``.  C is written in place.
"""

import torch

from ..registry import get_kernel
from .base_op import Op


class GemvOp(Op):
    _params_desc = {
        "N": "Number of columns of C",
        "K": "Reduction dimension (A cols, B rows)",
    }
    _atol = 1e-2
    _rtol = 1e-2

    def __init__(self, N: int, K: int, backend: str = "ref"):
        self.N, self.K = N, K
        self._backend = backend
        self._kernel = self._ref_forward if backend == "ref" else get_kernel("gemv", backend)(N=N, K=K)

    def forward(self, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor) -> None:
        self._kernel(A, B, C)

    def gen_data(self, device="cuda"):
        kw = dict(device=device, dtype=torch.bfloat16)
        A = torch.randn(self.K, **kw)
        b_shape = (self.K, self.N) if self._backend == "ref" else (self.N, self.K)
        B = torch.randn(*b_shape, **kw)
        C = torch.empty(self.N, **kw)
        return A, B, C

    def _ref_forward(self, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor) -> None:
        C.copy_(A @ B)
