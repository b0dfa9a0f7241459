"""A stack of Qwen3 dense decoder layers, one decode step (batch x 1 token).

The step either side of the reference's single-layer operator: its layer leaves
out RoPE and norm weights on purpose (ezops/ops/qwen3_dense_decode.py:27-29) and
its README lists the model loop as not implemented (README.md:16).  Here layer
``l`` is the reference layer formula (ezops/ops/qwen3_dense_decode.py:142-176)
with, optionally,

* weights on the input / post-attention RMSNorms (as in
  ezops/ops/fused_o_proj_ffn.py:107-110) and on the q / k head norms, and
* the rotary embedding of the new token's q and k, computed as the stand-alone
  operator does (ezops/ops/fused_qk_norm_rope.py:138-147: head norm, weight and
  rotate-half in fp32, one bf16 rounding) with the table row of ``position``;

* per-row lengths (``seq_lens``, each in 1..seq_len): row b's new token goes to cache slot
  ``seq_lens[b] - 1``, attends to its first ``seq_lens[b]`` keys and is rotated with the table
  row of that slot - the per-row position of sequences of different lengths in one batch
  (the reference's attention and RoPE operators each take one length / position for all rows);

and feeds layer ``l + 1``.  ``gen_data`` returns ``(hidden, layers, cos, sin)``
where ``layers`` is a list of dicts of bf16 tensors: ``K_cache``, ``V_cache``
[B, NKV, S, D] (slot S-1 receives the new k / v), ``Wqkv``, ``Wo``, ``Wgu``,
``Wd`` and the four norm weights (``None`` = unit).  ``cos`` / ``sin`` are the
reference's [max_seq_len, D] tables or ``None``.  Rounding differences between
two correct implementations add up along the residual stream, so the
acceptance bound is the layer's 1e-2 relative Frobenius error times
sqrt(num_layers).
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..registry import get_kernel
from .base_op import Op, rel_frobenius

NORM_KEYS = ("input_norm_w", "post_norm_w", "q_norm_w", "k_norm_w")


class Qwen3DecodeStackOp(Op):
    _params_desc = {
        "batch": "Batch size (tokens per decode step)",
        "seq_len": "KV cache length; the last slot holds the token being decoded",
        "hidden_size": "Hidden dimension",
        "intermediate_size": "MLP intermediate dimension",
        "num_heads": "Number of query heads",
        "head_dim": "Dimension per head",
        "num_layers": "Number of decoder layers",
        "num_kv_heads": "Number of KV heads for GQA (default: num_heads)",
        "rope": "1 = rotary embedding at position seq_len - 1 (default), 0 = none",
        "norm_weights": "1 = random norm weights 1 + N(0, 0.1) (default), 0 = unit weights",
        "seq_lens": "optional list of per-row lengths in 1..seq_len (default: every row has seq_len)",
    }
    _rtol = 1e-2
    rms_eps = 1e-6
    rope_theta = 1e6

    def __init__(self, batch, seq_len, hidden_size, intermediate_size, num_heads, head_dim, num_layers, backend="ref",
                 num_kv_heads=None, rope=1, norm_weights=1, seq_lens=None):
        if seq_len < 1 or num_layers < 1:
            raise ValueError(f"seq_len ({seq_len}) and num_layers ({num_layers}) must be >= 1")
        self.batch, self.seq_len, self.num_layers = batch, seq_len, num_layers
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_heads, self.head_dim = num_heads, head_dim
        self.num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        if num_heads % self.num_kv_heads != 0:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({self.num_kv_heads})")
        self.rope, self.norm_weights = bool(rope), bool(norm_weights)
        self.position = seq_len - 1
        if seq_lens is not None:
            seq_lens = [int(v) for v in seq_lens]
            if len(seq_lens) != batch or any(v < 1 or v > seq_len for v in seq_lens):
                raise ValueError(f"seq_lens must hold {batch} values in [1, {seq_len}]")
        self.seq_lens = seq_lens
        self._lens_dev = None
        self.q_rows, self.kv_rows = num_heads * head_dim, self.num_kv_heads * head_dim
        self._backend = backend
        if backend == "ref":
            self._kernel = self._ref_forward
        else:
            self._kernel = get_kernel("qwen3_decode_stack", backend)(
                batch, seq_len, hidden_size, intermediate_size, num_heads, head_dim, num_layers, num_kv_heads=self.num_kv_heads)

    def check(self, actual, expected) -> bool:
        bound = self._rtol * math.sqrt(self.num_layers)
        return actual.shape == expected.shape and rel_frobenius(actual, expected) < bound

    def forward(self, hidden, layers, cos=None, sin=None):
        if self._backend == "ref" or self.seq_lens is None:
            return self._kernel(hidden, layers, cos, sin)
        if self._lens_dev is None or self._lens_dev.device != hidden.device:
            self._lens_dev = torch.tensor(self.seq_lens, dtype=torch.int32, device=hidden.device)
        return self._kernel(hidden, layers, cos, sin, seq_lens=self._lens_dev)

    def rope_tables(self, device):
        """ezops/ops/fused_qk_norm_rope.py:119-125."""
        D = self.head_dim
        inv_freq = 1.0 / (self.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32, device=device) / D))
        ang = torch.arange(self.seq_len, dtype=torch.float32, device=device)[:, None] * inv_freq[None, :]
        return (torch.cat([ang.cos(), ang.cos()], dim=-1).to(torch.bfloat16),
                torch.cat([ang.sin(), ang.sin()], dim=-1).to(torch.bfloat16))

    def gen_data(self, device="cuda"):
        kw = dict(device=device, dtype=torch.bfloat16)
        B, S, H, I, D = self.batch, self.seq_len, self.hidden_size, self.intermediate_size, self.head_dim
        hidden = torch.randn(B, H, **kw)
        layers = []
        for _ in range(self.num_layers):
            layer = {
                "K_cache": torch.randn(B, self.num_kv_heads, S, D, **kw), "V_cache": torch.randn(B, self.num_kv_heads, S, D, **kw),
                "Wqkv": torch.randn(self.q_rows + 2 * self.kv_rows, H, **kw) * H**-0.5, "Wo": torch.randn(H, self.q_rows, **kw) * self.q_rows**-0.5,
                "Wgu": torch.randn(2 * I, H, **kw) * H**-0.5, "Wd": torch.randn(H, I, **kw) * I**-0.5,
            }
            for key, n in zip(NORM_KEYS, (H, H, D, D)):
                layer[key] = (1.0 + 0.1 * torch.randn(n, device=device)).to(torch.bfloat16) if self.norm_weights else None
            layers.append(layer)
        cos, sin = self.rope_tables(device) if self.rope else (None, None)
        return hidden, layers, cos, sin

    def _rmsnorm(self, x, w=None):
        y = x * torch.rsqrt(x.to(torch.float32).pow(2).mean(-1, keepdim=True) + self.rms_eps)
        return (y if w is None else y * w).to(x.dtype)

    def _head(self, x, w, c, s):
        """Head norm (+ weight) (+ rotation); fp32 throughout when rotating, one rounding."""
        if c is None:
            return self._rmsnorm(x, w)
        xf = x.to(torch.float32)
        n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.rms_eps)
        if w is not None:
            n = n * w.to(torch.float32)
        h = n.shape[-1] // 2
        rot = torch.cat((-n[..., h:], n[..., :h]), dim=-1)
        return (n * c + rot * s).to(torch.bfloat16)

    def _ref_forward(self, hidden, layers, cos=None, sin=None):
        B, D, I = hidden.shape[0], self.head_dim, self.intermediate_size
        q_end, k_end = self.q_rows, self.q_rows + self.kv_rows
        lens = self.seq_lens if self.seq_lens is not None else [self.seq_len] * B
        pos = torch.tensor([n - 1 for n in lens], device=hidden.device)
        c = cos[pos].to(torch.float32)[:, None, :] if cos is not None else None  # [B, 1, D]: one table row per batch row
        s = sin[pos].to(torch.float32)[:, None, :] if sin is not None else None
        rows = torch.arange(B, device=hidden.device)
        x_in = hidden
        for L in layers:
            qkv = self._rmsnorm(x_in, L.get("input_norm_w")) @ L["Wqkv"].T
            q = self._head(qkv[:, :q_end].view(B, self.num_heads, D), L.get("q_norm_w"), c, s)
            k = self._head(qkv[:, q_end:k_end].view(B, self.num_kv_heads, D), L.get("k_norm_w"), c, s)
            L["K_cache"][rows, :, pos, :] = k
            L["V_cache"][rows, :, pos, :] = qkv[:, k_end:].view(B, self.num_kv_heads, D)
            if self.seq_lens is None:
                attn = F.scaled_dot_product_attention(q.unsqueeze(2), L["K_cache"], L["V_cache"], enable_gqa=True).squeeze(2)
            else:  # every row attends to its own prefix
                attn = torch.cat([F.scaled_dot_product_attention(q[b : b + 1].unsqueeze(2), L["K_cache"][b : b + 1, :, :n],
                                                                 L["V_cache"][b : b + 1, :, :n], enable_gqa=True).squeeze(2)
                                  for b, n in enumerate(lens)], dim=0)
            x2 = x_in + attn.reshape(B, self.q_rows) @ L["Wo"].T
            gu = self._rmsnorm(x2, L.get("post_norm_w")) @ L["Wgu"].T
            x_in = x2 + (F.silu(gu[:, :I]) * gu[:, I:]) @ L["Wd"].T
        return x_in

    def get_roofline(self):
        raise NotImplementedError("use algorithmic bytes: num_layers x (layer weights + KV cache)")
