"""Seeded synthetic workloads at the Qwen3 shapes the benchmarks and parity
tests run on.  Tensors are drawn on the CPU from one ``torch.Generator`` in a
fixed order and then moved to the requested device, so a CPU check and a GPU
kernel always see identical bits.

Distributions: activations and KV entries N(0, 1); projection weights
N(0, 0.02); norm weights 1 + N(0, 0.1); RoPE tables for theta = 1e6.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

BF16 = torch.bfloat16


@dataclass(frozen=True)
class LayerShape:
    name: str
    hidden: int
    inter: int
    num_heads: int
    num_kv_heads: int
    head_dim: int

    @property
    def q_rows(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_rows(self) -> int:
        return self.num_kv_heads * self.head_dim

    def weight_bytes(self) -> int:
        H, I = self.hidden, self.inter
        return 2 * ((self.q_rows + 2 * self.kv_rows) * H + H * self.q_rows + 2 * I * H + H * I)

    def kv_bytes(self, batch: int, seq_len: int) -> int:
        return 2 * 2 * batch * self.num_kv_heads * seq_len * self.head_dim

    def algorithmic_bytes(self, batch: int, seq_len: int, tp: int = 1) -> int:
        return (self.weight_bytes() + self.kv_bytes(batch, seq_len)) // tp


QWEN3_8B = LayerShape("qwen3-8b", 4096, 12288, 32, 8, 128)
QWEN3_32B = LayerShape("qwen3-32b", 5120, 25600, 64, 8, 128)
QWEN3_VL_2B = LayerShape("qwen3-vl-2b", 2048, 6144, 16, 8, 128)
QWEN3_0_6B = LayerShape("qwen3-0.6b", 1024, 3072, 16, 8, 128)


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def _randn(g, *shape, std: float = 1.0, mean: float = 0.0) -> torch.Tensor:
    t = torch.randn(*shape, generator=g, dtype=torch.float32)
    if std != 1.0:
        t = t * std
    if mean != 0.0:
        t = t + mean
    return t.to(BF16)


def gemv_inputs(N: int = 4096, K: int = 4096, seed: int = 42, device="cpu"):
    """x [K] ~ N(0,1); W [N,K] ~ N(0,0.02); y [N] empty."""
    g = _gen(seed)
    x = _randn(g, K)
    W = _randn(g, N, K, std=0.02)
    y = torch.empty(N, dtype=BF16)
    return tuple(t.to(device) for t in (x, W, y))


def rmsnorm_inputs(rows: int = 32, dim: int = 4096, seed: int = 42, device="cpu"):
    g = _gen(seed)
    X = _randn(g, rows, dim)
    w = _randn(g, dim, std=0.1, mean=1.0)
    return X.to(device), w.to(device)


def rope_tables(max_seq_len: int, head_dim: int, theta: float = 1e6):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.arange(max_seq_len, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([ang.cos(), ang.cos()], -1).to(BF16), torch.cat([ang.sin(), ang.sin()], -1).to(BF16)


def qk_norm_rope_inputs(batch=32, num_heads=32, num_kv_heads=8, head_dim=128, max_seq_len=8192, seed=42, device="cpu"):
    """Returns (tensors in operator order, positions list)."""
    g = _gen(seed)
    q = _randn(g, batch, num_heads, head_dim)
    k = _randn(g, batch, num_kv_heads, head_dim)
    v = _randn(g, batch, num_kv_heads, head_dim)
    qw = _randn(g, head_dim, std=0.1, mean=1.0)
    kw = _randn(g, head_dim, std=0.1, mean=1.0)
    cos, sin = rope_tables(max_seq_len, head_dim)
    Kc = _randn(g, batch, num_kv_heads, max_seq_len, head_dim)
    Vc = _randn(g, batch, num_kv_heads, max_seq_len, head_dim)
    positions = torch.randint(0, max_seq_len, (batch,), generator=g).tolist()
    return tuple(t.to(device) for t in (q, k, v, qw, kw, cos, sin, Kc, Vc)), positions


def attn_decode_inputs(batch=32, num_heads=32, num_kv_heads=8, head_dim=128, max_len=8192, min_len=1024, seed=42,
                       device="cpu"):
    """Returns ((Q, K, V), seq_lens) with lengths uniform in [min_len, max_len]."""
    g = _gen(seed)
    lens = torch.randint(min_len, max_len + 1, (batch,), generator=g).tolist()
    Q = _randn(g, batch, num_heads, 1, head_dim)
    K = _randn(g, batch, num_kv_heads, max_len, head_dim)
    V = _randn(g, batch, num_kv_heads, max_len, head_dim)
    return tuple(t.to(device) for t in (Q, K, V)), lens


def layer_weights(shape: LayerShape, seed: int = 42, std: float = 0.02, device="cpu"):
    g = _gen(seed)
    H, I = shape.hidden, shape.inter
    Wqkv = _randn(g, shape.q_rows + 2 * shape.kv_rows, H, std=std)
    Wo = _randn(g, H, shape.q_rows, std=std)
    Wgu = _randn(g, 2 * I, H, std=std)
    Wd = _randn(g, H, I, std=std)
    return tuple(t.to(device) for t in (Wqkv, Wo, Wgu, Wd))


def layer_activations(shape: LayerShape, batch: int, seq_len: int, seed: int = 43, device="cpu"):
    g = _gen(seed)
    hidden = _randn(g, batch, shape.hidden)
    Kc = _randn(g, batch, shape.num_kv_heads, seq_len, shape.head_dim)
    Vc = _randn(g, batch, shape.num_kv_heads, seq_len, shape.head_dim)
    return tuple(t.to(device) for t in (hidden, Kc, Vc))


def decode_layer_inputs(shape: LayerShape, batch: int, seq_len: int, seed: int = 42, device="cpu"):
    """(hidden, K_cache, V_cache, Wqkv, Wo, Wgu, Wd) in operator order."""
    return layer_activations(shape, batch, seq_len, seed + 1, device) + layer_weights(shape, seed, device=device)


def decode_stack_inputs(shape: LayerShape, batch: int, seq_len: int, num_layers: int, rope: bool = True, norm_weights: bool = True,
                        seed: int = 42, device="cpu"):
    """(hidden, layers, cos, sin) for ``Qwen3DecodeStackOp``: every layer has its own seeded
    weights N(0, 0.02) and KV cache N(0, 1); norm weights 1 + N(0, 0.1); the reference's rotary tables."""
    g = _gen(seed + 7)
    hidden = _randn(g, batch, shape.hidden).to(device)
    layers = []
    for l in range(num_layers):
        Wqkv, Wo, Wgu, Wd = layer_weights(shape, seed + 100 * (l + 1), device=device)
        _, Kc, Vc = layer_activations(shape, batch, seq_len, seed + 100 * (l + 1) + 1, device=device)
        layer = {"K_cache": Kc, "V_cache": Vc, "Wqkv": Wqkv, "Wo": Wo, "Wgu": Wgu, "Wd": Wd}
        for key, n in (("input_norm_w", shape.hidden), ("post_norm_w", shape.hidden), ("q_norm_w", shape.head_dim), ("k_norm_w", shape.head_dim)):
            layer[key] = _randn(g, n, std=0.1, mean=1.0).to(device) if norm_weights else None
        layers.append(layer)
    cos, sin = (t.to(device) for t in rope_tables(seq_len, shape.head_dim)) if rope else (None, None)
    return hidden, layers, cos, sin


def o_proj_ffn_inputs(shape: LayerShape, batch: int, seed: int = 42, device="cpu"):
    g = _gen(seed)
    H, I, Q = shape.hidden, shape.inter, shape.q_rows
    attn = _randn(g, batch, Q)
    residual = _randn(g, batch, H)
    Wo = _randn(g, H, Q, std=0.02)
    pw = _randn(g, H, std=0.1, mean=1.0)
    Wg = _randn(g, I, H, std=0.02)
    Wu = _randn(g, I, H, std=0.02)
    Wd = _randn(g, H, I, std=0.02)
    return tuple(t.to(device) for t in (attn, residual, Wo, pw, Wg, Wu, Wd))
