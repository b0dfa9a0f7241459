"""ezops_b200: the Qwen3 dense-decode path of ez-ops as hand-written sm_100a
kernels behind ez-ops' own operator / registry API."""

from . import kernels as _kernels  # noqa: F401  (registers the backends; needs libezb200.so)
from .ops import (
    AttnDecodeOp,
    FusedOProjFfnOp,
    FusedQkNormRopeOp,
    GemvOp,
    Op,
    PdlGemmOp,
    Qwen3DecodeStackOp,
    Qwen3DenseDecodeOp,
    ReduceOp,
    RmsNormOp,
    RooflineResult,
    SoftmaxOp,
    VectorAddOp,
)
from .registry import get_kernel, list_backends, list_ops, register_kernel

__all__ = [
    "AttnDecodeOp",
    "FusedOProjFfnOp",
    "FusedQkNormRopeOp",
    "GemvOp",
    "Op",
    "PdlGemmOp",
    "Qwen3DecodeStackOp",
    "Qwen3DenseDecodeOp",
    "ReduceOp",
    "RmsNormOp",
    "RooflineResult",
    "SoftmaxOp",
    "VectorAddOp",
    "get_kernel",
    "list_backends",
    "list_ops",
    "register_kernel",
]
