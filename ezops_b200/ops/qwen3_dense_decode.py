"""One decode step of a Qwen3 dense decoder layer, batch x 1 token
(ezops/ops/qwen3_dense_decode.py:9-176)::

    x        = rmsnorm(hidden)                       # unit weight, eps 1e-6
    q, k, v  = x @ Wqkv.T                            # fused rows [q | k | v]
    q, k     = rmsnorm(q), rmsnorm(k)                # per head over head_dim
    K_cache[:, :, -1] = k ; V_cache[:, :, -1] = v    # new token -> last slot
    attn     = GQA(q, K_cache, V_cache) / sqrt(D)
    x2       = hidden + attn @ Wo.T
    out      = x2 + (silu(g) * u) @ Wd.T,  [g | u] = rmsnorm(x2) @ Wgu.T

RoPE is left out by the reference on purpose (qwen3_dense_decode.py:27-29).
Tensors in ``gen_data`` order, all bf16: hidden [B, H]; K_cache, V_cache
[B, NKV, S, D] (slot S-1 is scratch on input, the new k / v on output);
Wqkv [(NH+2*NKV)*D, H]; Wo [H, NH*D]; Wgu [2*I, H] rows [gate | up]; Wd [H, I].
Acceptance is relative Frobenius error < 1e-2 (qwen3_dense_decode.py:64-69).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ..registry import get_kernel
from .base_op import Op, rel_frobenius


class Qwen3DenseDecodeOp(Op):
    _params_desc = {
        "batch": "Batch size (tokens per decode step)",
        "seq_len": "KV cache length; the last slot holds the token being decoded",
        "hidden_size": "Hidden dimension",
        "intermediate_size": "MLP intermediate dimension",
        "num_heads": "Number of query heads",
        "head_dim": "Dimension per head",
        "num_kv_heads": "Number of KV heads for GQA (default: num_heads)",
    }
    _atol = 1e-2
    _rtol = 1e-2
    rms_eps = 1e-6

    def __init__(
        self,
        batch: int,
        seq_len: int,
        hidden_size: int,
        intermediate_size: int,
        num_heads: int,
        head_dim: int,
        backend: str = "ref",
        num_kv_heads: int | None = None,
    ):
        if seq_len < 1:
            raise ValueError(f"seq_len ({seq_len}) must be >= 1")
        self.batch, self.seq_len = batch, seq_len
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_heads, self.head_dim = num_heads, head_dim
        self.num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        if num_heads % self.num_kv_heads != 0:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({self.num_kv_heads})")
        self.q_rows = num_heads * head_dim
        self.kv_rows = self.num_kv_heads * head_dim
        self._backend = backend
        if backend == "ref":
            self._kernel = self._ref_forward
        else:
            self._kernel = get_kernel("qwen3_dense_decode", backend)(
                batch, seq_len, hidden_size, intermediate_size, num_heads, head_dim, num_kv_heads=self.num_kv_heads
            )

    def check(self, actual, expected) -> bool:
        return actual.shape == expected.shape and rel_frobenius(actual, expected) < self._rtol

    def forward(self, hidden, K_cache, V_cache, Wqkv, Wo, Wgu, Wd):
        return self._kernel(hidden, K_cache, V_cache, Wqkv, Wo, Wgu, Wd)

    def gen_data(self, device="cuda"):
        kw = dict(device=device, dtype=torch.bfloat16)
        B, S, H, I = self.batch, self.seq_len, self.hidden_size, self.intermediate_size
        hidden = torch.randn(B, H, **kw)
        K_cache = torch.randn(B, self.num_kv_heads, S, self.head_dim, **kw)
        V_cache = torch.randn(B, self.num_kv_heads, S, self.head_dim, **kw)
        Wqkv = torch.randn(self.q_rows + 2 * self.kv_rows, H, **kw) * H**-0.5
        Wo = torch.randn(H, self.q_rows, **kw) * self.q_rows**-0.5
        Wgu = torch.randn(2 * I, H, **kw) * H**-0.5
        Wd = torch.randn(H, I, **kw) * I**-0.5
        return hidden, K_cache, V_cache, Wqkv, Wo, Wgu, Wd

    def _rmsnorm(self, x):
        var = x.to(torch.float32).pow(2).mean(-1, keepdim=True)
        return (x * torch.rsqrt(var + self.rms_eps)).to(x.dtype)

    def _ref_forward(self, hidden, K_cache, V_cache, Wqkv, Wo, Wgu, Wd):
        B, D = hidden.shape[0], self.head_dim
        q_end, k_end = self.q_rows, self.q_rows + self.kv_rows

        qkv = self._rmsnorm(hidden) @ Wqkv.T
        q = self._rmsnorm(qkv[:, :q_end].view(B, self.num_heads, D))
        k = self._rmsnorm(qkv[:, q_end:k_end].view(B, self.num_kv_heads, D))
        v = qkv[:, k_end:].view(B, self.num_kv_heads, D)
        K_cache[:, :, -1, :] = k
        V_cache[:, :, -1, :] = v

        attn = F.scaled_dot_product_attention(q.unsqueeze(2), K_cache, V_cache, enable_gqa=True).squeeze(2)
        x2 = hidden + attn.reshape(B, self.q_rows) @ Wo.T

        gu = self._rmsnorm(x2) @ Wgu.T
        gate, up = gu[:, : self.intermediate_size], gu[:, self.intermediate_size :]
        return x2 + (F.silu(gate) * up) @ Wd.T
