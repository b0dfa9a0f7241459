"""CPU oracle for the Qwen3 dense-decode hot path.

TEST INFRASTRUCTURE, NOT PRODUCT.  Each function restates, on torch CPU
tensors, the algorithm of one reference ``_ref_forward`` (file:line cited per
function, paths relative to the reference project root) with the reference's
own staging: bf16 storage, every matmul result rounded to bf16, norm statistics
in fp32.  The arithmetic itself is PyTorch's (``@``, ``rsqrt``, ``F.silu``,
SDPA; the reference pins torch 2.12.0 in uv.lock, this image has 2.11.0).

Pinning: the reference holds no golden vectors for this path (its tests compare
backends against these same torch formulas), so the oracle is pinned against
outputs of the reference's own ``_ref_forward`` methods, generated once by
``tests/golden/make_golden.py`` (which imports the reference package) and
committed under ``tests/golden/``; ``tests/test_oracle_golden.py`` replays them.

Two kinds of function live here:
  * ``*_ref``   -- the reference's staging, used for parity;
  * ``*_fp64``  -- the same mathematics in float64 without intermediate
                   rounding, used to tell "kernel differs from the bf16-staged
                   reference" apart from "kernel is wrong".
Extensions the reference does not have (per-row positions, per-sequence
lengths, bf16 RMSNorm with weight, tensor-parallel sharding) apply the
reference's formula row by row / shard by shard and say so.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

RMS_EPS = 1e-6
ROPE_THETA = 1e6


# ---------------------------------------------------------------- GEMV ------
def gemv_ref(x: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    """y[N] = W[N,K] . x[K]; bf16 in/out (ezops/ops/gemv.py:37-38 computes
    ``A @ B`` with B = W.T as [K, N]; the layouts differ, the sums do not)."""
    return x @ W.T.contiguous()


def gemv_fp32(x: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    """fp32-accumulated result before the final bf16 rounding."""
    return W.to(torch.float32) @ x.to(torch.float32)


# ------------------------------------------------------------- RMSNorm ------
def rmsnorm_f32_ref(X: torch.Tensor, eps: float = RMS_EPS) -> torch.Tensor:
    """fp32, no weight (ezops/ops/rmsnorm.py:34-36)."""
    ms = X.pow(2).mean(dim=-1, keepdim=True)
    return X * torch.rsqrt(ms + eps)


def rmsnorm_bf16_ref(X: torch.Tensor, w: torch.Tensor | None = None, eps: float = RMS_EPS) -> torch.Tensor:
    """bf16 rows, fp32 statistics, optional bf16 weight, one rounding
    (ezops/ops/fused_o_proj_ffn.py:107-110 with weight;
    ezops/ops/qwen3_dense_decode.py:137-140 without)."""
    var = X.to(torch.float32).pow(2).mean(-1, keepdim=True)
    y = X * torch.rsqrt(var + eps)
    if w is not None:
        y = y * w
    return y.to(X.dtype)


# ----------------------------------------------------- QK-norm + RoPE -------
def rope_tables(max_seq_len: int, head_dim: int, theta: float = ROPE_THETA):
    """HF-layout bf16 cos/sin tables, halves repeated
    (ezops/ops/fused_qk_norm_rope.py:119-125)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.arange(max_seq_len, dtype=torch.float32)[:, None] * inv_freq[None, :]
    cos = torch.cat([ang.cos(), ang.cos()], dim=-1).to(torch.bfloat16)
    sin = torch.cat([ang.sin(), ang.sin()], dim=-1).to(torch.bfloat16)
    return cos, sin


def _head_norm_f32(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    # ezops/ops/fused_qk_norm_rope.py:138-141 -- result stays fp32
    xf = x.to(torch.float32)
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.to(torch.float32)


def _rotate_half_f32(x: torch.Tensor, c: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    # ezops/ops/fused_qk_norm_rope.py:143-147
    h = x.shape[-1] // 2
    rot = torch.cat((-x[..., h:], x[..., :h]), dim=-1)
    return (x * c + rot * s).to(torch.bfloat16)


def qk_norm_rope_ref(q, k, v, qw, kw, cos, sin, K_cache, V_cache, position, eps: float = RMS_EPS):
    """ezops/ops/fused_qk_norm_rope.py:149-169.  ``position`` is an int (the
    reference's case) or one int per batch row (extension: same formula per
    row).  Mutates the caches in place; returns (q_out, k_out)."""
    B = q.shape[0]
    pos = [position] * B if isinstance(position, int) else [int(p) for p in position]
    idx = torch.tensor(pos)
    c = cos[idx].to(torch.float32)[:, None, :]
    s = sin[idx].to(torch.float32)[:, None, :]
    q_out = _rotate_half_f32(_head_norm_f32(q, qw, eps), c, s)
    k_out = _rotate_half_f32(_head_norm_f32(k, kw, eps), c, s)
    for b, p in enumerate(pos):
        K_cache[b, :, p, :] = k_out[b]
        V_cache[b, :, p, :] = v[b]
    return q_out, k_out


# ------------------------------------------------------ decode attention ----
def attn_decode_ref(Q, K, V, seq_lens=None) -> torch.Tensor:
    """softmax(Q K^T / sqrt(D)) V for one query token, GQA by head grouping
    (ezops/ops/attn_decode.py:64-67; the cuDNN-only restriction there is dropped
    because it cannot run on CPU -- SDPA's math is backend independent).
    ``seq_lens`` (extension): per-row valid length, applied by slicing."""
    if seq_lens is None:
        return F.scaled_dot_product_attention(Q, K, V, enable_gqa=True)
    outs = []
    for b, n in enumerate(seq_lens):
        n = int(n)
        outs.append(F.scaled_dot_product_attention(Q[b : b + 1], K[b : b + 1, :, :n], V[b : b + 1, :, :n], enable_gqa=True))
    return torch.cat(outs, dim=0)


def attn_decode_fp64(Q, K, V, seq_lens=None) -> torch.Tensor:
    """Same function in float64 from the definition (no SDPA), [B, H, 1, D]."""
    B, H, _, D = Q.shape
    NKV = K.shape[1]
    G = H // NKV
    out = torch.empty(B, H, 1, D, dtype=torch.float64)
    for b in range(B):
        n = K.shape[2] if seq_lens is None else int(seq_lens[b])
        Kb = K[b, :, :n].to(torch.float64).repeat_interleave(G, dim=0)  # [H, n, D]
        Vb = V[b, :, :n].to(torch.float64).repeat_interleave(G, dim=0)
        s = torch.einsum("hd,hnd->hn", Q[b, :, 0].to(torch.float64), Kb) / (D**0.5)
        out[b, :, 0] = torch.einsum("hn,hnd->hd", torch.softmax(s, dim=-1), Vb)
    return out


# ------------------------------------------------------ o_proj + FFN --------
def o_proj_ffn_ref(attn, residual, Wo, post_norm_w, Wg, Wu, Wd, eps: float = RMS_EPS) -> torch.Tensor:
    """ezops/ops/fused_o_proj_ffn.py:112-125."""
    x2 = residual + attn @ Wo.T
    xn = rmsnorm_bf16_ref(x2, post_norm_w, eps)
    gate, up = xn @ Wg.T, xn @ Wu.T
    return x2 + (F.silu(gate) * up) @ Wd.T


def o_proj_ffn_fp64(attn, residual, Wo, post_norm_w, Wg, Wu, Wd, eps: float = RMS_EPS) -> torch.Tensor:
    d = torch.float64
    x2 = residual.to(d) + attn.to(d) @ Wo.to(d).T
    xn = x2 * torch.rsqrt(x2.pow(2).mean(-1, keepdim=True) + eps) * post_norm_w.to(d)
    return x2 + (F.silu(xn @ Wg.to(d).T) * (xn @ Wu.to(d).T)) @ Wd.to(d).T


# ------------------------------------------------------ the decode layer ----
def gqa_decode_attention_by_kv_head(q: torch.Tensor, K_cache: torch.Tensor, V_cache: torch.Tensor) -> torch.Tensor:
    """softmax(q K^T / sqrt(D)) V for one query token with grouped queries, one kv head at a time in fp32 and
    rounded to bf16 once: the same function as ``F.scaled_dot_product_attention(q[:, :, None], K, V,
    enable_gqa=True)`` (ezops/ops/qwen3_dense_decode.py:166-170) without materialising K and V once per query head,
    which at Qwen3-32B, batch 64, 8192 keys would be 2 x 17 GB.  q [B, NH, D], caches [B, NKV, S, D] -> [B, NH, D]."""
    B, NH, D = q.shape
    NKV = K_cache.shape[1]
    G = NH // NKV
    out = torch.empty(B, NH, D, dtype=q.dtype)
    scale = 1.0 / (D**0.5)
    for h in range(NKV):
        qg = q[:, h * G : (h + 1) * G].float()                      # [B, G, D]
        scores = torch.einsum("bgd,bsd->bgs", qg, K_cache[:, h].float()) * scale
        probs = torch.softmax(scores, dim=-1)
        out[:, h * G : (h + 1) * G] = torch.einsum("bgs,bsd->bgd", probs, V_cache[:, h].float()).to(q.dtype)
    return out


def qwen3_dense_decode_ref(hidden, K_cache, V_cache, Wqkv, Wo, Wgu, Wd, num_heads, num_kv_heads, head_dim,
                           eps: float = RMS_EPS, sdpa_math: bool = False, lean_attention: bool = False) -> torch.Tensor:
    """ezops/ops/qwen3_dense_decode.py:142-176.  Mutates slot S-1 of the caches.

    The reference restricts SDPA to [cuDNN, MATH] (qwen3_dense_decode.py:167).
    On its home device that selects cuDNN (fp32 scores and softmax); on CPU
    tensors it selects the MATH path, which keeps scores and softmax in bf16.
    ``sdpa_math=True`` reproduces the CPU selection literally (this is what the
    golden fixtures were generated through); the default leaves the backend
    free, which on CPU picks the fused kernel with fp32 softmax -- the staging
    the reference has on a GPU and the one GPU kernels are compared with.
    ``lean_attention=True`` computes that attention one kv head at a time (see
    gqa_decode_attention_by_kv_head), for shapes whose expanded K/V would not fit."""
    B = hidden.shape[0]
    q_rows, kv_rows = num_heads * head_dim, num_kv_heads * head_dim
    inter = Wgu.shape[0] // 2

    x = rmsnorm_bf16_ref(hidden, None, eps)
    qkv = x @ Wqkv.T
    q = rmsnorm_bf16_ref(qkv[:, :q_rows].view(B, num_heads, head_dim), None, eps)
    k = rmsnorm_bf16_ref(qkv[:, q_rows : q_rows + kv_rows].view(B, num_kv_heads, head_dim), None, eps)
    v = qkv[:, q_rows + kv_rows :].view(B, num_kv_heads, head_dim)
    K_cache[:, :, -1, :] = k
    V_cache[:, :, -1, :] = v

    if lean_attention:  # large shapes: the same attention without a copy of K and V per query head
        attn = gqa_decode_attention_by_kv_head(q, K_cache, V_cache)
    elif sdpa_math:
        from torch.nn.attention import SDPBackend, sdpa_kernel

        with sdpa_kernel([SDPBackend.MATH]):
            attn = F.scaled_dot_product_attention(q.unsqueeze(2), K_cache, V_cache, enable_gqa=True).squeeze(2)
    else:
        attn = F.scaled_dot_product_attention(q.unsqueeze(2), K_cache, V_cache, enable_gqa=True).squeeze(2)
    x2 = hidden + attn.reshape(B, q_rows) @ Wo.T

    gu = rmsnorm_bf16_ref(x2, None, eps) @ Wgu.T
    gate, up = gu[:, :inter], gu[:, inter:]
    return x2 + (F.silu(gate) * up) @ Wd.T


def qwen3_dense_decode_fp64(hidden, K_cache, V_cache, Wqkv, Wo, Wgu, Wd, num_heads, num_kv_heads, head_dim,
                            eps: float = RMS_EPS) -> torch.Tensor:
    """Float64 layer without intermediate rounding; does not touch the caches
    (the new k/v are spliced into float64 copies)."""
    d = torch.float64
    B = hidden.shape[0]
    q_rows, kv_rows = num_heads * head_dim, num_kv_heads * head_dim
    inter = Wgu.shape[0] // 2

    def norm(t):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)

    h = hidden.to(d)
    qkv = norm(h) @ Wqkv.to(d).T
    q = norm(qkv[:, :q_rows].view(B, num_heads, head_dim))
    k = norm(qkv[:, q_rows : q_rows + kv_rows].view(B, num_kv_heads, head_dim))
    v = qkv[:, q_rows + kv_rows :].view(B, num_kv_heads, head_dim)
    Kc, Vc = K_cache.to(d).clone(), V_cache.to(d).clone()
    Kc[:, :, -1, :] = k
    Vc[:, :, -1, :] = v
    G = num_heads // num_kv_heads
    s = torch.einsum("bhd,bhnd->bhn", q, Kc.repeat_interleave(G, dim=1)) / (head_dim**0.5)
    attn = torch.einsum("bhn,bhnd->bhd", torch.softmax(s, -1), Vc.repeat_interleave(G, dim=1))
    x2 = h + attn.reshape(B, q_rows) @ Wo.to(d).T
    gu = norm(x2) @ Wgu.to(d).T
    return x2 + (F.silu(gu[:, :inter]) * gu[:, inter:]) @ Wd.to(d).T


# ------------------------------------------------ tensor-parallel sharding ---
def qwen3_decode_stack_ref(hidden, layers, num_heads, num_kv_heads, head_dim, cos=None, sin=None, position=None,
                           eps: float = RMS_EPS, seq_lens=None) -> torch.Tensor:
    """A stack of decode layers: the layer formula above (ezops/ops/qwen3_dense_decode.py:142-176)
    per layer, each feeding the next.  Optional per-layer norm weights (``None`` = unit; weighted
    RMSNorm as ezops/ops/fused_o_proj_ffn.py:107-110) and, when ``cos`` / ``sin`` are given, the
    new token's q and k go through the stand-alone operator's formula (``_head_norm_f32`` +
    ``_rotate_half_f32``, ezops/ops/fused_qk_norm_rope.py:138-147) with the table row of
    ``position`` (default S-1).  ``layers``: dicts with K_cache, V_cache (slot S-1 is written),
    Wqkv, Wo, Wgu, Wd and optionally input_norm_w, post_norm_w, q_norm_w, k_norm_w.
    ``seq_lens`` (one int per batch row, 1..S): row b's token goes to slot seq_lens[b]-1, attends to
    its first seq_lens[b] keys (per-row SDPA over the prefix, as ``attn_decode_ref`` does for ragged
    batches) and is rotated with that slot's table row (per-row positions, as ``qk_norm_rope_ref``).
    No single reference function covers this composition; each piece is pinned by its own fixtures."""
    B = hidden.shape[0]
    q_rows, kv_rows = num_heads * head_dim, num_kv_heads * head_dim
    x_in = hidden
    for L in layers:
        S = L["K_cache"].shape[2]
        if seq_lens is not None:
            slots = [int(n) - 1 for n in seq_lens]
        else:
            slots = [S - 1 if position is None else position] * B
        lens = [int(n) for n in seq_lens] if seq_lens is not None else [S] * B
        inter = L["Wgu"].shape[0] // 2
        qkv = rmsnorm_bf16_ref(x_in, L.get("input_norm_w"), eps) @ L["Wqkv"].T
        q = qkv[:, :q_rows].view(B, num_heads, head_dim)
        k = qkv[:, q_rows : q_rows + kv_rows].view(B, num_kv_heads, head_dim)
        v = qkv[:, q_rows + kv_rows :].view(B, num_kv_heads, head_dim)
        if cos is None:
            q = rmsnorm_bf16_ref(q, L.get("q_norm_w"), eps)
            k = rmsnorm_bf16_ref(k, L.get("k_norm_w"), eps)
        else:
            ones = torch.ones(head_dim, dtype=torch.bfloat16)
            idx = torch.tensor(slots)
            c, s = cos[idx].to(torch.float32)[:, None, :], sin[idx].to(torch.float32)[:, None, :]
            qw = ones if L.get("q_norm_w") is None else L["q_norm_w"]
            kw = ones if L.get("k_norm_w") is None else L["k_norm_w"]
            q = _rotate_half_f32(_head_norm_f32(q, qw, eps), c, s)
            k = _rotate_half_f32(_head_norm_f32(k, kw, eps), c, s)
        for b, slot in enumerate(slots):
            L["K_cache"][b, :, slot, :] = k[b]
            L["V_cache"][b, :, slot, :] = v[b]
        if seq_lens is None:
            attn = F.scaled_dot_product_attention(q.unsqueeze(2), L["K_cache"], L["V_cache"], enable_gqa=True).squeeze(2)
        else:
            attn = torch.cat([F.scaled_dot_product_attention(q[b : b + 1].unsqueeze(2), L["K_cache"][b : b + 1, :, :n],
                                                             L["V_cache"][b : b + 1, :, :n], enable_gqa=True).squeeze(2)
                              for b, n in enumerate(lens)], dim=0)
        x2 = x_in + attn.reshape(B, q_rows) @ L["Wo"].T
        gu = rmsnorm_bf16_ref(x2, L.get("post_norm_w"), eps) @ L["Wgu"].T
        x_in = x2 + (F.silu(gu[:, :inter]) * gu[:, inter:]) @ L["Wd"].T
    return x_in


def shard_layer_weights(Wqkv, Wo, Wgu, Wd, num_heads, num_kv_heads, head_dim, tp: int, rank: int):
    """Megatron-style split of one layer's weights for rank ``rank`` of ``tp``
    (no reference counterpart: the reference is single-GPU).  q heads and kv
    heads are split contiguously; Wo keeps the columns of the rank's q heads;
    gate/up rows and Wd columns are split contiguously."""
    assert num_kv_heads % tp == 0 and num_heads % tp == 0
    D = head_dim
    q_rows, kv_rows = num_heads * D, num_kv_heads * D
    inter = Wgu.shape[0] // 2
    assert inter % tp == 0
    ql, kl, il = q_rows // tp, kv_rows // tp, inter // tp
    q = Wqkv[rank * ql : (rank + 1) * ql]
    k = Wqkv[q_rows + rank * kl : q_rows + (rank + 1) * kl]
    v = Wqkv[q_rows + kv_rows + rank * kl : q_rows + kv_rows + (rank + 1) * kl]
    Wqkv_r = torch.cat([q, k, v], dim=0).contiguous()
    Wo_r = Wo[:, rank * ql : (rank + 1) * ql].contiguous()
    Wgu_r = torch.cat([Wgu[rank * il : (rank + 1) * il], Wgu[inter + rank * il : inter + (rank + 1) * il]], dim=0).contiguous()
    Wd_r = Wd[:, rank * il : (rank + 1) * il].contiguous()
    return Wqkv_r, Wo_r, Wgu_r, Wd_r


def shard_kv_cache(cache, tp: int, rank: int):
    nkv = cache.shape[1] // tp
    return cache[:, rank * nkv : (rank + 1) * nkv].contiguous()


# ---- the reference's teaching operators (CPU, float64 accumulation: an oracle independent of any GPU result) ----
def vector_add_ref(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """C = A + B in fp32 (ezops/ops/vector_add.py:29-30)."""
    return A.cpu() + B.cpu()


def softmax_ref(X: torch.Tensor) -> torch.Tensor:
    """Row soft-max (ezops/ops/softmax.py:35-36), computed in float64 and rounded to fp32 once."""
    return torch.softmax(X.cpu().double(), dim=-1).float()


def reduce_sum_ref(A: torch.Tensor) -> torch.Tensor:
    """Sum of all elements (ezops/ops/reduce.py:32-33), accumulated in float64."""
    return A.cpu().double().sum().float().reshape(1)


def pdl_gemm_ref(x: torch.Tensor, W1: torch.Tensor, W2: torch.Tensor):
    """y = x @ W1, z = y @ W2 (ezops/ops/pdl_gemm.py:69-76), accumulated in float64 and rounded to fp32 once per
    GEMM: (y, z)."""
    y = (x.cpu().double() @ W1.cpu().double()).float()
    z = (y.double() @ W2.cpu().double()).float()
    return y, z
