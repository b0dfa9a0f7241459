"""Post-attention tail of a Qwen3 dense decoder layer, batch x 1 token
(ezops/ops/fused_o_proj_ffn.py:8-125)::

    x2  = residual + attn @ Wo.T
    xn  = rmsnorm(x2) * post_norm_w                      # eps 1e-6
    out = x2 + (silu(xn @ Wg.T) * (xn @ Wu.T)) @ Wd.T

Tensors in ``gen_data`` order, all bf16: attn [B, NH*D], residual [B, H],
Wo [H, NH*D], post_norm_w [H], Wg [I, H], Wu [I, H], Wd [H, I].  The o_proj
input width NH*D is independent of H (Qwen3-0.6B: 2048 lanes into hidden 1024).
Acceptance is relative Frobenius error < 1e-2 (fused_o_proj_ffn.py:51-56)
because the torch reference rounds every stage to bf16.
"""

import torch
import torch.nn.functional as F

from ..registry import get_kernel
from .base_op import Op, rel_frobenius


class FusedOProjFfnOp(Op):
    _params_desc = {
        "batch": "Batch size (tokens per decode step)",
        "hidden_size": "Hidden dimension",
        "intermediate_size": "MLP intermediate dimension",
        "num_heads": "Number of query heads (o_proj input width = num_heads * head_dim)",
        "head_dim": "Dimension per head",
    }
    _atol = 1e-2
    _rtol = 1e-2
    rms_eps = 1e-6

    def __init__(self, batch, hidden_size, intermediate_size, num_heads, head_dim, backend: str = "ref"):
        self.batch, self.hidden_size, self.intermediate_size = batch, hidden_size, intermediate_size
        self.num_heads, self.head_dim = num_heads, head_dim
        self.q_rows = num_heads * head_dim
        self._backend = backend
        if backend == "ref":
            self._kernel = self._ref_forward
        else:
            self._kernel = get_kernel("fused_o_proj_ffn", backend)(
                batch, hidden_size, intermediate_size, num_heads, head_dim
            )

    def check(self, actual, expected) -> bool:
        return actual.shape == expected.shape and rel_frobenius(actual, expected) < self._rtol

    def forward(self, attn, residual, Wo, post_norm_w, Wg, Wu, Wd):
        return self._kernel(attn, residual, Wo, post_norm_w, Wg, Wu, Wd)

    def gen_data(self, device="cuda"):
        kw = dict(device=device, dtype=torch.bfloat16)
        H, I, Q, B = self.hidden_size, self.intermediate_size, self.q_rows, self.batch
        attn = torch.randn(B, Q, **kw)
        residual = torch.randn(B, H, **kw)
        Wo = torch.randn(H, Q, **kw) * Q**-0.5  # fan-in scaling keeps activations O(1)
        post_norm_w = torch.randn(H, **kw)
        Wg = torch.randn(I, H, **kw) * H**-0.5
        Wu = torch.randn(I, H, **kw) * H**-0.5
        Wd = torch.randn(H, I, **kw) * I**-0.5
        return attn, residual, Wo, post_norm_w, Wg, Wu, Wd

    def _rmsnorm(self, x, w):
        var = x.to(torch.float32).pow(2).mean(-1, keepdim=True)
        return (x * torch.rsqrt(var + self.rms_eps) * w).to(x.dtype)

    def _ref_forward(self, attn, residual, Wo, post_norm_w, Wg, Wu, Wd):
        x2 = residual + attn @ Wo.T
        xn = self._rmsnorm(x2, post_norm_w)
        return x2 + (F.silu(xn @ Wg.T) * (xn @ Wu.T)) @ Wd.T
