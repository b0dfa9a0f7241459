from .attn_decode import AttnDecodeOp
from .base_op import Op
from .fused_o_proj_ffn import FusedOProjFfnOp
from .fused_qk_norm_rope import FusedQkNormRopeOp
from .gemv import GemvOp
from .qwen3_decode_stack import Qwen3DecodeStackOp
from .qwen3_dense_decode import Qwen3DenseDecodeOp
from .rmsnorm import RmsNormOp
from .tutorial import PdlGemmOp, ReduceOp, SoftmaxOp, VectorAddOp
from .utils.roofline import RooflineResult

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
]
