"""Roofline accounting for an op's torch reference (ezops/ops/utils/roofline.py:54-88).

``measure_roofline`` runs a callable under torch's FLOP counter, with an extra
table so that element-wise ops count one flop per output element and ``mv``
counts 2*M*K (the stock counter ignores both), and sums the byte sizes of every
tensor argument plus every returned tensor.  ``algorithmic_bytes_*`` helpers
give the "each tensor once, intermediates on chip" byte counts that the
HBM-roofline fractions of this package are quoted against.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
from torch.utils.flop_counter import FlopCounterMode

_aten = torch.ops.aten


def _numel(shape) -> int:
    return math.prod(shape)


def _one_flop_per_output(*_in_shapes, out_shape=None, **_kw) -> int:
    return _numel(out_shape) if out_shape is not None else 0


def _mat_vec(*in_shapes, out_shape=None, **_kw) -> int:
    if len(in_shapes) < 2 or len(in_shapes[0]) != 2:
        return 0
    rows, cols = in_shapes[0]
    return 2 * rows * cols


_POINTWISE = (
    "add sub mul div neg abs exp log sqrt rsqrt relu sigmoid tanh silu gelu pow "
    "copy clone where maximum minimum"
).split()

_CUSTOM_FLOPS = {getattr(_aten, name): _one_flop_per_output for name in _POINTWISE}
_CUSTOM_FLOPS[_aten.mv] = _mat_vec


@dataclass(frozen=True)
class RooflineResult:
    flops: int
    bytes: int
    fused_bytes: int
    arithmetic_intensity: float = field(default=0.0)

    def __post_init__(self):
        ai = self.flops / self.bytes if self.bytes > 0 else float("inf")
        object.__setattr__(self, "arithmetic_intensity", ai)


def _tensor_bytes(obj) -> int:
    if isinstance(obj, torch.Tensor):
        return obj.nbytes
    if isinstance(obj, (tuple, list)):
        return sum(t.nbytes for t in obj if isinstance(t, torch.Tensor))
    return 0


def measure_roofline(fn, args: tuple, kwargs: dict) -> RooflineResult:
    with FlopCounterMode(display=False, custom_mapping=_CUSTOM_FLOPS) as counter:
        result = fn(*args, **kwargs)
    nbytes = _tensor_bytes(list(args)) + _tensor_bytes(list(kwargs.values())) + _tensor_bytes(result)
    return RooflineResult(flops=counter.get_total_flops(), bytes=nbytes, fused_bytes=nbytes)


# --------------------------------------------------------------------------
# Algorithmic byte counts (every weight and every valid KV row read once,
# activations in/out once, on-chip intermediates not counted).  bf16 = 2 bytes.
# --------------------------------------------------------------------------

def algorithmic_bytes_gemv(N: int, K: int) -> int:
    return 2 * (N * K + K + N)


def algorithmic_bytes_attn_decode(total_kv_len: int, batch: int, num_heads: int, num_kv_heads: int, head_dim: int) -> int:
    """``total_kv_len`` is the sum of the per-sequence valid lengths."""
    kv = total_kv_len * num_kv_heads * head_dim * 2 * 2
    q_and_out = 2 * batch * num_heads * head_dim * 2
    return kv + q_and_out


def algorithmic_bytes_decode_layer(
    batch: int, seq_len: int, hidden: int, inter: int, num_heads: int, head_dim: int, num_kv_heads: int, tp: int = 1
) -> int:
    """Weights + KV cache + the [batch, hidden] activation in and out, per GPU
    when the heads / FFN columns are split ``tp`` ways."""
    q_rows, kv_rows = num_heads * head_dim, num_kv_heads * head_dim
    weights = 2 * ((q_rows + 2 * kv_rows) * hidden + hidden * q_rows + 2 * inter * hidden + hidden * inter)
    kv = 2 * 2 * batch * num_kv_heads * seq_len * head_dim
    return (weights + kv) // tp


def algorithmic_bytes_o_proj_ffn(batch: int, hidden: int, inter: int, q_rows: int) -> int:
    weights = 2 * (hidden * q_rows + 3 * inter * hidden + hidden)
    acts = 2 * batch * (q_rows + 2 * hidden)
    return weights + acts
