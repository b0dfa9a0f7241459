"""RMSNorm operator spec (ezops/ops/rmsnorm.py:7-36).

The reference op is fp32 without a weight: ``Out = X * rsqrt(mean(X^2) + eps)``.
Extension used by the Qwen3 configurations: ``dtype=torch.bfloat16`` with
``with_weight=True`` adds a per-dim bf16 weight and follows the staging of the
layer norms inside the fused ops (ezops/ops/fused_o_proj_ffn.py:107-110):
statistics in fp32, ``x * rsqrt(var + eps) * w`` in fp32, one rounding to bf16.
In that mode ``forward``/``gen_data`` carry the weight as a third tensor:
``(X, W, Out)``.
"""

import torch

from ..registry import get_kernel
from .base_op import Op


class RmsNormOp(Op):
    _params_desc = {
        "batch_size": "Number of rows",
        "dim": "Feature dimension per row (normalized over dim)",
    }
    _atol = 1e-5
    _rtol = 1e-5

    def __init__(
        self,
        batch_size: int,
        dim: int,
        backend: str = "ref",
        eps: float = 1e-6,
        dtype: torch.dtype = torch.float32,
        with_weight: bool = False,
    ):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"dtype must be float32 or bfloat16, got {dtype}")
        if with_weight and dtype != torch.bfloat16:
            raise ValueError("with_weight=True is the bf16 Qwen3 variant; use dtype=torch.bfloat16")
        self.batch_size, self.dim, self.eps = batch_size, dim, eps
        self.dtype, self.with_weight = dtype, with_weight
        self._backend = backend
        if dtype == torch.bfloat16:
            self._atol = self._rtol = 1e-2
        if backend == "ref":
            self._kernel = self._ref_forward
        else:
            extra = {} if (dtype == torch.float32 and not with_weight) else dict(dtype=dtype, with_weight=with_weight)
            self._kernel = get_kernel("rmsnorm", backend)(batch_size=batch_size, dim=dim, eps=eps, **extra)

    def forward(self, X: torch.Tensor, *rest: torch.Tensor) -> None:
        self._kernel(X, *rest)

    def gen_data(self, device="cuda"):
        X = torch.randn(self.batch_size, self.dim, device=device, dtype=self.dtype)
        Out = torch.empty_like(X)
        if self.with_weight:
            W = (1.0 + 0.1 * torch.randn(self.dim, device=device)).to(self.dtype)
            return X, W, Out
        return X, Out

    def _ref_forward(self, X: torch.Tensor, *rest: torch.Tensor) -> None:
        if self.with_weight:
            W, Out = rest
            var = X.to(torch.float32).pow(2).mean(dim=-1, keepdim=True)
            Out.copy_((X * torch.rsqrt(var + self.eps) * W).to(X.dtype))
            return
        (Out,) = rest
        if X.dtype == torch.float32:
            ms = X.pow(2).mean(dim=-1, keepdim=True)
            Out.copy_(X * torch.rsqrt(ms + self.eps))
        else:
            var = X.to(torch.float32).pow(2).mean(dim=-1, keepdim=True)
            Out.copy_((X * torch.rsqrt(var + self.eps)).to(X.dtype))
