"""The sm_100a backends: one kernel class per operator of the decode path,
registered as backend ``"cuda"``.  Each class validates what the operator
contract asks of a constructor (``ValueError`` naming the rule), owns its
workspace, and forwards to one entry point of ``libezb200.so`` on torch's
current stream.  Calls enqueue work only (no synchronisation, no allocation
after the first call), so they can be captured in a CUDA graph.
"""

from __future__ import annotations

import torch

from .. import _lib
from ..registry import register_kernel
from .base_kernel import BaseKernel

_BF16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require(t: torch.Tensor, name: str, shape, dtype=_BF16) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _zeros_bytes(nbytes: int, device) -> torch.Tensor:
    return torch.zeros(max(int(nbytes), 256), dtype=torch.uint8, device=device)


@register_kernel("gemv", "cuda")
class GemvSm100Kernel(BaseKernel):
    """C[N] = B[N,K] . A[K] (constructor contract: ezops/ops/gemv.py:21)."""

    def __init__(self, N: int, K: int):
        if K % 16:
            raise ValueError(f"K ({K}) must be divisible by 16")
        self.N, self.K = N, K
        self._lib = _lib.load()

    def __call__(self, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor) -> None:
        _require(A, "A", (self.K,))
        _require(B, "B", (self.N, self.K))
        _require(C, "C", (self.N,))
        _lib.check(self._lib.ezb_gemv_bf16(A.data_ptr(), B.data_ptr(), C.data_ptr(), self.N, self.K, _stream()))


@register_kernel("rmsnorm", "cuda")
class RmsNormSm100Kernel(BaseKernel):
    """fp32 rows without weight (ezops/ops/rmsnorm.py:22), or the bf16 variant
    with optional weight when constructed with ``dtype=torch.bfloat16``."""

    def __init__(self, batch_size: int, dim: int, eps: float = 1e-6, dtype=torch.float32, with_weight: bool = False):
        if dtype == _BF16 and dim % 8:
            raise ValueError(f"dim ({dim}) must be divisible by 8 for bf16 rows")
        self.rows, self.dim, self.eps, self.dtype, self.with_weight = batch_size, dim, eps, dtype, with_weight
        self._lib = _lib.load()

    def __call__(self, X: torch.Tensor, *rest: torch.Tensor) -> None:
        shape = (self.rows, self.dim)
        if self.dtype == torch.float32:
            (Out,) = rest
            _require(X, "X", shape, torch.float32)
            _require(Out, "Out", shape, torch.float32)
            _lib.check(self._lib.ezb_rmsnorm_f32(X.data_ptr(), Out.data_ptr(), self.rows, self.dim, self.eps, _stream()))
            return
        if self.with_weight:
            W, Out = rest
            _require(W, "W", (self.dim,))
        else:
            (Out,), W = rest, None
        _require(X, "X", shape)
        _require(Out, "Out", shape)
        _lib.check(
            self._lib.ezb_rmsnorm_bf16(
                X.data_ptr(), W.data_ptr() if W is not None else None, Out.data_ptr(), self.rows, self.dim, self.eps, _stream()
            )
        )


@register_kernel("fused_qk_norm_rope", "cuda")
class FusedQkNormRopeSm100Kernel(BaseKernel):
    """Constructor contract: ezops/ops/fused_qk_norm_rope.py:85-92.  ``position``
    may be a list with one entry per batch row (extension)."""

    rms_eps = 1e-6

    def __init__(self, batch, num_heads, head_dim, max_seq_len, position, num_kv_heads=None):
        self.B, self.NQ, self.D, self.S = batch, num_heads, head_dim, max_seq_len
        self.NKV = num_heads if num_kv_heads is None else num_kv_heads
        if head_dim & (head_dim - 1) or not 8 <= head_dim <= 512:
            raise ValueError(f"head_dim ({head_dim}) must be a power of two in [8, 512]")
        if num_heads % self.NKV:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({self.NKV})")
        self.position = position
        self._positions_dev = None
        self._lib = _lib.load()

    def __call__(self, q, k, v, q_norm_w, k_norm_w, cos, sin, K_cache, V_cache):
        B, NQ, NKV, D, S = self.B, self.NQ, self.NKV, self.D, self.S
        _require(q, "q", (B, NQ, D)); _require(k, "k", (B, NKV, D)); _require(v, "v", (B, NKV, D))
        _require(q_norm_w, "q_norm_w", (D,)); _require(k_norm_w, "k_norm_w", (D,))
        _require(cos, "cos", (S, D)); _require(sin, "sin", (S, D))
        _require(K_cache, "K_cache", (B, NKV, S, D)); _require(V_cache, "V_cache", (B, NKV, S, D))
        q_out, k_out = torch.empty_like(q), torch.empty_like(k)
        if isinstance(self.position, int):
            pos, pos_ptr = self.position, None
        else:
            if self._positions_dev is None or self._positions_dev.device != q.device:
                self._positions_dev = torch.tensor(list(self.position), dtype=torch.int32, device=q.device)
            pos, pos_ptr = 0, self._positions_dev.data_ptr()
        _lib.check(
            self._lib.ezb_qk_norm_rope(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), q_norm_w.data_ptr(), k_norm_w.data_ptr(), cos.data_ptr(),
                sin.data_ptr(), K_cache.data_ptr(), V_cache.data_ptr(), q_out.data_ptr(), k_out.data_ptr(),
                B, NQ, NKV, D, S, pos, pos_ptr, self.rms_eps, _stream(),
            )
        )
        return q_out, k_out


@register_kernel("attn_decode", "cuda")
class AttnDecodeSm100Kernel(BaseKernel):
    """Split-KV GQA flash decode (constructor contract: ezops/ops/attn_decode.py:42-51)."""

    supports_gqa = True

    def __init__(self, batch, num_heads, seq_len, head_dim, num_kv_heads=None, seq_lens=None):
        self.B, self.H, self.S, self.D = batch, num_heads, seq_len, head_dim
        self.NKV = num_heads if num_kv_heads is None else num_kv_heads
        if head_dim not in (64, 128):
            raise ValueError(f"head_dim ({head_dim}) must be 64 or 128")
        if num_heads % self.NKV:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({self.NKV})")
        self.seq_lens = None if seq_lens is None else [int(x) for x in seq_lens]
        self._lens_dev = None
        self._ws = None
        self._lib = _lib.load()

    def _workspace(self, device):
        need = self._lib.ezb_attn_decode_workspace_bytes(self.B, self.H, self.NKV, self.S, self.D)
        if self._ws is None or self._ws.device != device or self._ws.numel() < need:
            self._ws = _zeros_bytes(need, device)
        return self._ws

    def __call__(self, Q, K, V):
        B, H, NKV, S, D = self.B, self.H, self.NKV, self.S, self.D
        _require(Q, "Q", (B, H, 1, D)); _require(K, "K", (B, NKV, S, D)); _require(V, "V", (B, NKV, S, D))
        out = torch.empty_like(Q)
        ws = self._workspace(Q.device)
        lens_ptr = None
        if self.seq_lens is not None:
            if self._lens_dev is None or self._lens_dev.device != Q.device:
                self._lens_dev = torch.tensor(self.seq_lens, dtype=torch.int32, device=Q.device)
            lens_ptr = self._lens_dev.data_ptr()
        _lib.check(
            self._lib.ezb_attn_decode(
                Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(),
                B, H, NKV, S, D, lens_ptr, _stream(),
            )
        )
        return out

    def call_paged(self, Q, K_pool, V_pool, page_table, seq_lens, page_size):
        """The same attention over paged caches: ``K_pool`` / ``V_pool`` [pages, NKV, page_size, D],
        ``page_table`` [B, max_pages] int32 and ``seq_lens`` [B] int32 on the device; the constructor's
        ``seq_len`` must equal ``max_pages * page_size``."""
        B, H, NKV, D = self.B, self.H, self.NKV, self.D
        _require(Q, "Q", (B, H, 1, D))
        max_pages = page_table.shape[1]
        if self.S != max_pages * page_size:
            raise ValueError(f"seq_len ({self.S}) must equal max_pages * page_size ({max_pages} * {page_size})")
        _require(page_table, "page_table", (B, max_pages), dtype=torch.int32)
        _require(seq_lens, "seq_lens", (B,), dtype=torch.int32)
        for name, t in (("K_pool", K_pool), ("V_pool", V_pool)):
            _require(t, name, (t.shape[0], NKV, page_size, D))
        out = torch.empty_like(Q)
        ws = self._workspace(Q.device)
        _lib.check(
            self._lib.ezb_attn_decode_paged(
                Q.data_ptr(), K_pool.data_ptr(), V_pool.data_ptr(), page_table.data_ptr(), out.data_ptr(), ws.data_ptr(),
                ws.numel(), B, H, NKV, max_pages, page_size, D, K_pool.shape[0], seq_lens.data_ptr(), _stream(),
            )
        )
        return out


@register_kernel("fused_o_proj_ffn", "cuda")
class FusedOProjFfnSm100Kernel(BaseKernel):
    """Constructor contract: ezops/ops/fused_o_proj_ffn.py:78."""

    rms_eps = 1e-6

    def __init__(self, batch, hidden_size, intermediate_size, num_heads, head_dim):
        self.B, self.H, self.I, self.Q = batch, hidden_size, intermediate_size, num_heads * head_dim
        for name, val in (("hidden_size", self.H), ("intermediate_size", self.I), ("num_heads * head_dim", self.Q)):
            if val % 16:
                raise ValueError(f"{name} ({val}) must be divisible by 16")
        if not 1 <= batch <= 64:
            raise ValueError(f"batch ({batch}) must be in [1, 64]")
        self._ws = None
        self._lib = _lib.load()

    def __call__(self, attn, residual, Wo, post_norm_w, Wg, Wu, Wd):
        B, H, I, Q = self.B, self.H, self.I, self.Q
        _require(attn, "attn", (B, Q)); _require(residual, "residual", (B, H)); _require(Wo, "Wo", (H, Q))
        _require(post_norm_w, "post_norm_w", (H,)); _require(Wg, "Wg", (I, H)); _require(Wu, "Wu", (I, H))
        _require(Wd, "Wd", (H, I))
        if self._ws is None or self._ws.device != attn.device:
            self._ws = _zeros_bytes(self._lib.ezb_o_proj_ffn_workspace_bytes(B, H, I, Q), attn.device)
        out = torch.empty_like(residual)
        _lib.check(
            self._lib.ezb_o_proj_ffn(
                attn.data_ptr(), residual.data_ptr(), Wo.data_ptr(), post_norm_w.data_ptr(), Wg.data_ptr(), Wu.data_ptr(),
                Wd.data_ptr(), out.data_ptr(), self._ws.data_ptr(), self._ws.numel(), B, H, I, Q, self.rms_eps, _stream(),
            )
        )
        return out


@register_kernel("qwen3_dense_decode", "cuda")
class Qwen3DenseDecodeSm100Kernel(BaseKernel):
    """The whole decode layer as a chain of five kernels linked by programmatic
    dependent launch (constructor contract: ezops/ops/qwen3_dense_decode.py:100-108)."""

    rms_eps = 1e-6
    direct_host_output = True  # host step: the layer's last kernel writes the pinned result buffer itself (102.0 -> 99.8 us per step)

    def __init__(self, batch, seq_len, hidden_size, intermediate_size, num_heads, head_dim, num_kv_heads=None):
        self.B, self.S, self.H, self.I = batch, seq_len, hidden_size, intermediate_size
        self.NH, self.D = num_heads, head_dim
        self.NKV = num_heads if num_kv_heads is None else num_kv_heads
        if num_heads % self.NKV:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by num_kv_heads ({self.NKV})")
        if head_dim not in (64, 128):
            raise ValueError(f"head_dim ({head_dim}) must be 64 or 128")
        if num_heads // self.NKV > 16:
            raise ValueError("at most 16 query heads per kv head")
        for name, val in (("hidden_size", self.H), ("intermediate_size", self.I)):
            if val % 16:
                raise ValueError(f"{name} ({val}) must be divisible by 16")
        if not 1 <= batch <= 64:
            raise ValueError(f"batch ({batch}) must be in [1, 64]")
        self._ws = None
        self._lib = _lib.load()

    def workspace(self, device):
        if self._ws is None or self._ws.device != device:
            need = self._lib.ezb_qwen3_decode_layer_workspace_bytes(self.B, self.S, self.H, self.I, self.NH, self.NKV, self.D)
            self._ws = _zeros_bytes(need, device)
        return self._ws

    def _host_step(self, hidden, K_cache, V_cache, Wqkv, Wo, Wgu, Wd, out):
        """The step's input and result live in PINNED host memory: a copy-in kernel (``ezb_copy_pinned``) and the
        layer as one dependency chain on the current stream; the result goes to the host buffer either straight from
        the layer's last kernel (``direct_host_output``) or through a copy-out kernel.  ``out`` is valid once the
        stream is synchronised."""
        if not hidden.is_pinned() or hidden.dtype != _BF16 or tuple(hidden.shape) != (self.B, self.H) or not hidden.is_contiguous():
            raise ValueError(f"a host `hidden` must be a pinned contiguous bf16 tensor of shape {(self.B, self.H)}")
        if out is None:
            out = torch.empty_like(hidden).pin_memory()
        if out.is_cuda or not out.is_pinned() or out.dtype != _BF16 or tuple(out.shape) != (self.B, self.H) or not out.is_contiguous():
            raise ValueError("with a host `hidden`, `out` must be a pinned contiguous bf16 host tensor of the same shape")
        dev = K_cache.device
        if getattr(self, "_io", None) is None or self._io[0].device != dev:
            self._io = (torch.empty(self.B, self.H, dtype=_BF16, device=dev), torch.empty(self.B, self.H, dtype=_BF16, device=dev))
        d_in, d_out = self._io
        nbytes = self.B * self.H * 2
        _lib.check(self._lib.ezb_copy_pinned(d_in.data_ptr(), hidden.data_ptr(), nbytes, _stream()))
        if self.direct_host_output:
            # pinned host memory is device-addressable at the same address: the layer's last kernel stores the
            # result rows straight into it (a few hundred posted PCIe writes), no copy-out launch
            self(d_in, K_cache, V_cache, Wqkv, Wo, Wgu, Wd, out=out)
            return out
        self(d_in, K_cache, V_cache, Wqkv, Wo, Wgu, Wd, out=d_out)
        _lib.check(self._lib.ezb_copy_pinned(out.data_ptr(), d_out.data_ptr(), nbytes, _stream()))
        return out

    def __call__(self, hidden, K_cache, V_cache, Wqkv, Wo, Wgu, Wd, out=None):
        """``out`` (optional) receives the result in place.  ``hidden`` (and then ``out``) may be pinned host
        tensors: see ``_host_step``."""
        B, S, H, I, NH, NKV, D = self.B, self.S, self.H, self.I, self.NH, self.NKV, self.D
        if not hidden.is_cuda:
            return self._host_step(hidden, K_cache, V_cache, Wqkv, Wo, Wgu, Wd, out)
        _require(hidden, "hidden", (B, H))
        _require(K_cache, "K_cache", (B, NKV, S, D)); _require(V_cache, "V_cache", (B, NKV, S, D))
        _require(Wqkv, "Wqkv", ((NH + 2 * NKV) * D, H)); _require(Wo, "Wo", (H, NH * D))
        _require(Wgu, "Wgu", (2 * I, H)); _require(Wd, "Wd", (H, I))
        ws = self.workspace(hidden.device)
        if out is None:
            out = torch.empty_like(hidden)
        _lib.check(
            self._lib.ezb_qwen3_decode_layer(
                hidden.data_ptr(), K_cache.data_ptr(), V_cache.data_ptr(), Wqkv.data_ptr(), Wo.data_ptr(), Wgu.data_ptr(),
                Wd.data_ptr(), out.data_ptr(), ws.data_ptr(), ws.numel(), B, S, H, I, NH, NKV, D, self.rms_eps, _stream(),
            )
        )
        return out


@register_kernel("qwen3_decode_stack", "cuda")
class Qwen3DecodeStackSm100Kernel(BaseKernel):
    """``num_layers`` decode layers in one C call (``ezb_qwen3_decode_stack``): one chain of
    kernels through all layers, optional norm weights, RoPE inside the attention kernel.
    ``__call__(hidden, layers, cos, sin, out=None)`` with ``layers`` as described in
    ``ops/qwen3_decode_stack.py``.  The pointer table is rebuilt only when a tensor changes."""

    rms_eps = 1e-6

    def __init__(self, batch, seq_len, hidden_size, intermediate_size, num_heads, head_dim, num_layers, num_kv_heads=None):
        # same shape rules as one layer
        Qwen3DenseDecodeSm100Kernel.__init__(self, batch, seq_len, hidden_size, intermediate_size, num_heads, head_dim, num_kv_heads)
        if num_layers < 1:
            raise ValueError(f"num_layers ({num_layers}) must be >= 1")
        self.L = num_layers
        self._table, self._table_key = None, None

    def workspace(self, device):
        if self._ws is None or self._ws.device != device:
            need = self._lib.ezb_qwen3_decode_stack_workspace_bytes(self.B, self.S, self.H, self.I, self.NH, self.NKV, self.D)
            self._ws = _zeros_bytes(need, device)
        return self._ws

    def _layer_table(self, layers, page_size=None):
        B, S, H, I, NH, NKV, D = self.B, self.S, self.H, self.I, self.NH, self.NKV, self.D
        cache = (B, NKV, S, D) if page_size is None else (layers[0]["K_cache"].shape[0], NKV, page_size, D)  # pools when paged
        shapes = {"K_cache": cache, "V_cache": cache, "Wqkv": ((NH + 2 * NKV) * D, H), "Wo": (H, NH * D),
                  "Wgu": (2 * I, H), "Wd": (H, I), "input_norm_w": (H,), "post_norm_w": (H,), "q_norm_w": (D,), "k_norm_w": (D,)}
        key = tuple(0 if L.get(n) is None else L[n].data_ptr() for L in layers for n in shapes)
        if key != self._table_key:
            table = (_lib.LayerStruct * len(layers))()
            for i, L in enumerate(layers):
                for name, shape in shapes.items():
                    t = L.get(name)
                    if t is None:
                        if not name.endswith("_norm_w"):
                            raise ValueError(f"layer {i}: {name} is required")
                        setattr(table[i], name, None)
                        continue
                    _require(t, f"layer {i} {name}", shape)
                    setattr(table[i], name, t.data_ptr())
            self._table, self._table_key = table, key
        return self._table

    def __call__(self, hidden, layers, cos=None, sin=None, out=None, seq_lens=None, page_table=None, page_size=None):
        """``seq_lens`` (optional int32 CUDA tensor [B], values 1..S): row b's new token goes to slot
        ``seq_lens[b] - 1``, attends to its first ``seq_lens[b]`` keys and is rotated with that slot's table row.
        ``page_table`` ([B, max_pages] int32) + ``page_size``: the layers' K_cache / V_cache are page pools
        [pages, NKV, page_size, D]; needs ``seq_lens`` and ``S == max_pages * page_size``."""
        if len(layers) != self.L:
            raise ValueError(f"expected {self.L} layers, got {len(layers)}")
        _require(hidden, "hidden", (self.B, self.H))
        if (cos is None) != (sin is None):
            raise ValueError("cos and sin come as a pair")
        if seq_lens is not None:
            _require(seq_lens, "seq_lens", (self.B,), dtype=torch.int32)
        position = self.S - 1
        if cos is not None:
            for name, t in (("cos", cos), ("sin", sin)):
                if t.dim() != 2 or t.shape[1] != self.D or t.shape[0] <= position:
                    raise ValueError(f"{name} must be [> {position}, {self.D}], got {tuple(t.shape)}")
                _require(t, name, t.shape)
        if page_table is not None:
            if seq_lens is None or page_size is None:
                raise ValueError("paged caches need seq_lens and page_size")
            _require(page_table, "page_table", (self.B, page_table.shape[1]), dtype=torch.int32)
            if self.S != page_table.shape[1] * page_size:
                raise ValueError(f"seq_len ({self.S}) must equal max_pages * page_size")
            table = self._layer_table(layers, page_size)
            ws = self.workspace(hidden.device)
            if out is None:
                out = torch.empty_like(hidden)
            _lib.check(
                self._lib.ezb_qwen3_decode_stack_paged(
                    hidden.data_ptr(), out.data_ptr(), table, self.L, cos.data_ptr() if cos is not None else None,
                    sin.data_ptr() if sin is not None else None, seq_lens.data_ptr(), page_table.data_ptr(), page_size,
                    page_table.shape[1], layers[0]["K_cache"].shape[0], ws.data_ptr(), ws.numel(), self.B, self.H, self.I,
                    self.NH, self.NKV, self.D, self.rms_eps, _stream(),
                )
            )
            return out
        table = self._layer_table(layers)
        ws = self.workspace(hidden.device)
        if out is None:
            out = torch.empty_like(hidden)
        _lib.check(
            self._lib.ezb_qwen3_decode_stack(
                hidden.data_ptr(), out.data_ptr(), table, self.L, cos.data_ptr() if cos is not None else None,
                sin.data_ptr() if sin is not None else None, position, None if seq_lens is None else seq_lens.data_ptr(),
                ws.data_ptr(), ws.numel(), self.B, self.S, self.H, self.I, self.NH, self.NKV, self.D, self.rms_eps, _stream(),
            )
        )
        return out


# ------------------------------------------------------------ teaching operators ---
def _require_f32(t: torch.Tensor, name: str, shape) -> None:
    _require(t, name, shape, dtype=torch.float32)


@register_kernel("vector_add", "cuda")
class VectorAddSm100Kernel(BaseKernel):
    """C = A + B, fp32 (constructor contract: ezops/ops/vector_add.py:14-15)."""

    def __init__(self, n: int):
        if n < 1:
            raise ValueError(f"n ({n}) must be positive")
        self.n, self._lib = n, _lib.load()

    def __call__(self, A, B, C) -> None:
        for name, t in (("A", A), ("B", B), ("C", C)):
            _require_f32(t, name, (self.n,))
        _lib.check(self._lib.ezb_vector_add_f32(A.data_ptr(), B.data_ptr(), C.data_ptr(), self.n, _stream()))


@register_kernel("softmax", "cuda")
class SoftmaxSm100Kernel(BaseKernel):
    """Row softmax, fp32 (constructor contract: ezops/ops/softmax.py:19-20)."""

    def __init__(self, batch_size: int, dim: int):
        if batch_size < 1 or dim < 1:
            raise ValueError("batch_size and dim must be positive")
        self.rows, self.dim, self._lib = batch_size, dim, _lib.load()

    def __call__(self, X, Out) -> None:
        _require_f32(X, "X", (self.rows, self.dim)); _require_f32(Out, "Out", (self.rows, self.dim))
        _lib.check(self._lib.ezb_softmax_f32(X.data_ptr(), Out.data_ptr(), self.rows, self.dim, _stream()))


@register_kernel("reduce", "cuda")
class ReduceSm100Kernel(BaseKernel):
    """Sum of an fp32 vector into Out[0], bit-reproducible (constructor contract: ezops/ops/reduce.py:17-18)."""

    def __init__(self, n: int):
        if n < 1:
            raise ValueError(f"n ({n}) must be positive")
        self.n, self._lib, self._ws = n, _lib.load(), None

    def __call__(self, A, Out) -> None:
        _require_f32(A, "A", (self.n,)); _require_f32(Out, "Out", (1,))
        if self._ws is None or self._ws.device != A.device:
            self._ws = _zeros_bytes(self._lib.ezb_reduce_workspace_bytes(), A.device)
        _lib.check(self._lib.ezb_reduce_sum_f32(A.data_ptr(), Out.data_ptr(), self.n, self._ws.data_ptr(), self._ws.numel(), _stream()))



class _PdlGemmSm100Base(BaseKernel):
    """y = x @ W1, z = y @ W2 on fp32 tensors (constructor contract: ezops/ops/pdl_gemm.py:39-47; call contract
    ``(x, W1, W2, y, z) -> None`` as ezops/kernels/pdl_gemm/pdl_gemm_cu.py:34-42)."""

    use_pdl = 0

    def __init__(self, M: int, K: int, N: int, P: int):
        if min(M, K, N, P) < 1:
            raise ValueError("M, K, N and P must be positive")
        if K % 4 or N % 4 or P % 4:
            raise ValueError(f"K ({K}), N ({N}) and P ({P}) must be divisible by 4")
        self.M, self.K, self.N, self.P, self._lib = M, K, N, P, _lib.load()

    def __call__(self, x, W1, W2, y, z) -> None:
        M, K, N, P = self.M, self.K, self.N, self.P
        for name, t, shape in (("x", x, (M, K)), ("W1", W1, (K, N)), ("W2", W2, (N, P)), ("y", y, (M, N)), ("z", z, (M, P))):
            _require_f32(t, name, shape)
        _lib.check(self._lib.ezb_pdl_gemm_f32(x.data_ptr(), W1.data_ptr(), W2.data_ptr(), y.data_ptr(), z.data_ptr(),
                                              M, K, N, P, self.use_pdl, _stream()))


@register_kernel("pdl_gemm", "cuda")
class PdlGemmSm100Kernel(_PdlGemmSm100Base):
    """Two ordinary launches: the second GEMM starts when the first has finished."""

    use_pdl = 0


@register_kernel("pdl_gemm", "cuda_pdl")
class PdlGemmPdlSm100Kernel(_PdlGemmSm100Base):
    """The second GEMM is launched with programmatic stream serialization: its CTAs fetch their W2 tiles while the
    first GEMM drains and read y only after ``griddepcontrol.wait``."""

    use_pdl = 1
