"""Per-head QK RMSNorm + half-split RoPE + KV-cache slot write for one decode
step (ezops/ops/fused_qk_norm_rope.py:7-169).

For every query head and kv head of the token being decoded::

    q_out = rope(rmsnorm(q) * q_norm_w, cos[pos], sin[pos])
    k_out = rope(rmsnorm(k) * k_norm_w, cos[pos], sin[pos])
    K_cache[:, :, pos] = k_out ;  V_cache[:, :, pos] = v        (in place)

Norm through rotation stay in fp32 with a single rounding to bf16.  RoPE is the
rotate_half form against HF-layout tables [max_seq_len, head_dim] whose second
half repeats the first.  Tensors, in ``gen_data`` order (all bf16)::

    q [B, NQ, D]  k [B, NKV, D]  v [B, NKV, D]  q_norm_w [D]  k_norm_w [D]
    cos, sin [max_seq_len, D]    K_cache, V_cache [B, NKV, max_seq_len, D]

Extension over the reference (which has one scalar ``position`` for the whole
batch, fused_qk_norm_rope.py:66): ``position`` may also be a length-``batch``
sequence / tensor of ints, one RoPE row and one cache slot per batch row.
"""

from __future__ import annotations

import torch

from ..registry import get_kernel
from .base_op import Op


def _as_position_list(position, batch: int, max_seq_len: int):
    if isinstance(position, torch.Tensor):
        position = position.tolist()
    if isinstance(position, int):
        if not 0 <= position < max_seq_len:
            raise ValueError(f"position ({position}) must be in [0, {max_seq_len})")
        return position, None
    plist = [int(p) for p in position]
    if len(plist) != batch:
        raise ValueError(f"position has {len(plist)} entries for batch {batch}")
    for p in plist:
        if not 0 <= p < max_seq_len:
            raise ValueError(f"position ({p}) must be in [0, {max_seq_len})")
    return None, plist


class FusedQkNormRopeOp(Op):
    _params_desc = {
        "batch": "Batch size (tokens per decode step)",
        "num_heads": "Number of query heads",
        "head_dim": "Dimension per head (must be a power of two)",
        "max_seq_len": "KV cache capacity; also the cos/sin table length",
        "position": "Decode position: RoPE table row and cache slot to write (int, or one per batch row)",
        "num_kv_heads": "Number of KV heads for GQA (default: num_heads)",
    }
    _atol = 1e-2
    _rtol = 1e-2

    rms_eps = 1e-6
    rope_theta = 1e6

    def __init__(
        self,
        batch: int,
        num_heads: int,
        head_dim: int,
        max_seq_len: int,
        position,
        backend: str = "ref",
        num_kv_heads: int | None = None,
    ):
        if head_dim & (head_dim - 1):
            raise ValueError(f"head_dim ({head_dim}) must be a power of two")
        scalar, per_row = _as_position_list(position, batch, max_seq_len)
        self.batch, self.num_heads, self.head_dim, self.max_seq_len = batch, num_heads, head_dim, max_seq_len
        self.position = scalar if per_row is None else per_row
        self.num_kv_heads = num_heads if num_kv_heads is None else num_kv_heads
        if num_heads % self.num_kv_heads != 0:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({self.num_kv_heads})")
        self._backend = backend
        if backend == "ref":
            self._kernel = self._ref_forward
        else:
            self._kernel = get_kernel("fused_qk_norm_rope", backend)(
                batch, num_heads, head_dim, max_seq_len, self.position, num_kv_heads=self.num_kv_heads
            )

    def forward(self, q, k, v, q_norm_w, k_norm_w, cos, sin, K_cache, V_cache):
        return self._kernel(q, k, v, q_norm_w, k_norm_w, cos, sin, K_cache, V_cache)

    def rope_tables(self, device="cuda"):
        half = torch.arange(0, self.head_dim, 2, dtype=torch.float32, device=device) / self.head_dim
        inv_freq = 1.0 / (self.rope_theta**half)
        ang = torch.arange(self.max_seq_len, dtype=torch.float32, device=device)[:, None] * inv_freq[None, :]
        cos = torch.cat([ang.cos(), ang.cos()], dim=-1).to(torch.bfloat16)
        sin = torch.cat([ang.sin(), ang.sin()], dim=-1).to(torch.bfloat16)
        return cos, sin

    def gen_data(self, device="cuda"):
        kw = dict(device=device, dtype=torch.bfloat16)
        B, NQ, NKV, D, S = self.batch, self.num_heads, self.num_kv_heads, self.head_dim, self.max_seq_len
        q = torch.randn(B, NQ, D, **kw)
        k = torch.randn(B, NKV, D, **kw)
        v = torch.randn(B, NKV, D, **kw)
        q_norm_w = torch.randn(D, **kw)
        k_norm_w = torch.randn(D, **kw)
        cos, sin = self.rope_tables(device)
        K_cache = torch.randn(B, NKV, S, D, **kw)
        V_cache = torch.randn(B, NKV, S, D, **kw)
        return q, k, v, q_norm_w, k_norm_w, cos, sin, K_cache, V_cache

    def check(self, actual, expected) -> bool:
        if len(actual) != len(expected):
            return False
        return all(
            a.shape == e.shape and torch.allclose(a, e, atol=self._atol, rtol=self._rtol)
            for a, e in zip(actual, expected)
        )

    def _rmsnorm(self, x, w):
        xf = x.to(torch.float32)
        return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.rms_eps) * w.to(torch.float32)

    def _rope(self, x, cos_pos, sin_pos):
        h = self.head_dim // 2
        rotated = torch.cat((-x[..., h:], x[..., :h]), dim=-1)
        return (x * cos_pos + rotated * sin_pos).to(torch.bfloat16)

    def _ref_forward(self, q, k, v, q_norm_w, k_norm_w, cos, sin, K_cache, V_cache):
        if isinstance(self.position, int):
            c, s = cos[self.position].float(), sin[self.position].float()
            q_out = self._rope(self._rmsnorm(q, q_norm_w), c, s)
            k_out = self._rope(self._rmsnorm(k, k_norm_w), c, s)
            K_cache[:, :, self.position, :] = k_out
            V_cache[:, :, self.position, :] = v
            return q_out, k_out
        # one position per batch row: the same formula row by row
        pos = getattr(self, "_pos_cache", None)
        if pos is None or pos.device != q.device:  # kept on the device so the call can be graph-captured
            pos = self._pos_cache = torch.as_tensor(self.position, device=q.device)
        c, s = cos[pos].float()[:, None, :], sin[pos].float()[:, None, :]
        q_out = self._rope(self._rmsnorm(q, q_norm_w), c, s)
        k_out = self._rope(self._rmsnorm(k, k_norm_w), c, s)
        for b, p in enumerate(self.position):
            K_cache[b, :, p, :] = k_out[b]
            V_cache[b, :, p, :] = v[b]
        return q_out, k_out
