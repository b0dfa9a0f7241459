"""Single-query (decode) attention with GQA (ezops/ops/attn_decode.py:9-67).

``out = softmax(Q K^T / sqrt(D)) V`` for one query token per sequence:
Q [B, H, 1, D], K and V [B, NKV, S, D], out [B, H, 1, D], all bf16.  A kernel
class opts into grouped-query attention with the class attribute
``supports_gqa = True``; otherwise the op refuses ``num_kv_heads != num_heads``
(attn_decode.py:42-51).

Extension over the reference (one shared ``seq_len``): ``seq_lens`` gives one
valid length per sequence, 1 <= len <= seq_len; keys past a row's length are
not attended to (and not read).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ..registry import get_kernel
from .base_op import Op


class AttnDecodeOp(Op):
    _params_desc = {
        "batch": "Batch size",
        "num_heads": "Number of attention heads",
        "seq_len": "KV cache sequence length",
        "head_dim": "Dimension per head",
        "num_kv_heads": "Number of KV heads for GQA (default: num_heads)",
        "seq_lens": "Optional per-sequence valid lengths (default: all seq_len)",
    }
    _atol = 1e-2
    _rtol = 1e-2

    def __init__(
        self,
        batch: int,
        num_heads: int,
        seq_len: int,
        head_dim: int,
        backend: str = "ref",
        num_kv_heads: int | None = None,
        seq_lens=None,
    ):
        self.batch, self.num_heads, self.seq_len, self.head_dim = batch, num_heads, seq_len, head_dim
        self.num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        if num_heads % self.num_kv_heads != 0:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({self.num_kv_heads})")
        if seq_lens is not None:
            seq_lens = [int(x) for x in (seq_lens.tolist() if isinstance(seq_lens, torch.Tensor) else seq_lens)]
            if len(seq_lens) != batch or any(not 1 <= x <= seq_len for x in seq_lens):
                raise ValueError(f"seq_lens must hold {batch} values in [1, {seq_len}]")
        self.seq_lens = seq_lens
        self._backend = backend
        if backend == "ref":
            self._kernel = self._ref_forward
            return
        cls = get_kernel("attn_decode", backend)
        if getattr(cls, "supports_gqa", False):
            extra = {} if seq_lens is None else dict(seq_lens=seq_lens)
            self._kernel = cls(batch, num_heads, seq_len, head_dim, num_kv_heads=self.num_kv_heads, **extra)
        else:
            if self.num_kv_heads != num_heads:
                raise ValueError(
                    f"backend {backend!r} does not support GQA (num_kv_heads={self.num_kv_heads} != "
                    f"num_heads={num_heads}); expand K/V to num_heads before calling it"
                )
            self._kernel = cls(batch, num_heads, seq_len, head_dim)

    def forward(self, Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor) -> torch.Tensor:
        return self._kernel(Q, K, V)

    def gen_data(self, device="cuda"):
        kw = dict(device=device, dtype=torch.bfloat16)
        Q = torch.randn(self.batch, self.num_heads, 1, self.head_dim, **kw)
        K = torch.randn(self.batch, self.num_kv_heads, self.seq_len, self.head_dim, **kw)
        V = torch.randn(self.batch, self.num_kv_heads, self.seq_len, self.head_dim, **kw)
        return Q, K, V

    def _ref_forward(self, Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor) -> torch.Tensor:
        # The reference pins the cuDNN SDPA backend (attn_decode.py:65); any
        # SDPA backend computes the same function, so none is pinned here and
        # the reference also runs on CPU tensors.
        if self.seq_lens is None:
            return F.scaled_dot_product_attention(Q, K, V, enable_gqa=True)
        rows = [
            F.scaled_dot_product_attention(Q[b : b + 1], K[b : b + 1, :, :n], V[b : b + 1, :, :n], enable_gqa=True)
            for b, n in enumerate(self.seq_lens)
        ]
        return torch.cat(rows, dim=0)
