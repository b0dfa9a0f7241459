"""Host-side behaviour that needs no GPU: the registry, operator constructors,
the torch reference inside the operators, and the C-ABI library (it loads,
exports every declared symbol, and rejects bad arguments before touching CUDA).
"""

import ctypes
import re
from pathlib import Path

import pytest
import torch

import ezops_b200 as ez
from ezops_b200 import _lib
from ezops_b200.registry import get_kernel, list_backends, list_ops, register_kernel
from helpers import load_golden, rel_fro
from oracle import ezops_oracle as orc

ROOT = Path(__file__).resolve().parent.parent


def test_registry_lists_the_six_ops_with_a_cuda_backend():
    # the reference's six operators of the decode path, plus the multi-layer stack built on top of them
    assert list_ops() == sorted(["attn_decode", "fused_o_proj_ffn", "fused_qk_norm_rope", "gemv", "qwen3_decode_stack",
                                 "qwen3_dense_decode", "rmsnorm", "reduce", "softmax", "vector_add", "pdl_gemm"])
    for op in list_ops():
        assert "cuda" in list_backends(op)
        cls = get_kernel(op, "cuda")
        assert cls.op_name == op and cls.backend == "cuda"


def test_registry_duplicate_and_missing():
    with pytest.raises(ValueError, match="already registered"):
        register_kernel("gemv", "cuda")(type("Dup", (), {}))
    with pytest.raises(KeyError, match="Available backends"):
        get_kernel("gemv", "nope")

    @register_kernel("unit_test_op", "x")
    class K:  # noqa: D401
        def __call__(self):
            return 1

    assert get_kernel("unit_test_op", "x") is K and list_backends("unit_test_op") == ["x"]
    from ezops_b200 import registry

    del registry._REGISTRY[("unit_test_op", "x")]


def test_header_symbols_are_all_exported_and_bound():
    header = (ROOT / "include" / "ezb200.h").read_text()
    declared = set(re.findall(r"\b(ezb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in ezb200.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert lib.ezb_version() >= 100
    assert lib.ezb_strerror(0) == b"ok"


def test_c_abi_rejects_bad_arguments_without_a_gpu():
    lib = _lib.load()
    assert lib.ezb_gemv_bf16(None, None, None, 16, 16, None) == _lib.EZB_ERR_INVALID_ARGUMENT
    assert b"null" in lib.ezb_last_error_message()
    fake = ctypes.c_void_p(0x1000)
    assert lib.ezb_gemv_bf16(fake, fake, fake, 16, 100, None) == _lib.EZB_ERR_UNSUPPORTED_SHAPE
    assert lib.ezb_gemv_bf16(ctypes.c_void_p(0x1002), fake, fake, 16, 64, None) == _lib.EZB_ERR_INVALID_ARGUMENT
    assert lib.ezb_attn_decode(fake, fake, fake, fake, None, 0, 1, 8, 3, 128, 128, None, None) == _lib.EZB_ERR_UNSUPPORTED_SHAPE
    assert lib.ezb_attn_decode(fake, fake, fake, fake, None, 0, 1, 8, 2, 128, 128, None, None) == _lib.EZB_ERR_WORKSPACE
    # an output pointer that is only 2-byte aligned (a sliced view) is refused, not handed to 8-byte vector stores
    odd = ctypes.c_void_p(0x1002)
    assert lib.ezb_attn_decode(fake, fake, fake, odd, fake, 1 << 30, 1, 8, 2, 128, 128, None, None) == _lib.EZB_ERR_INVALID_ARGUMENT
    assert lib.ezb_attn_decode_paged(fake, fake, fake, fake, odd, fake, 1 << 30, 1, 8, 2, 2, 64, 128, 4, fake, None) == _lib.EZB_ERR_INVALID_ARGUMENT
    assert lib.ezb_attn_decode_static(fake, fake, fake, odd, 1, 8, 2, 128, 128, None, None) == _lib.EZB_ERR_INVALID_ARGUMENT
    assert lib.ezb_gemv_bf16(fake, fake, ctypes.c_void_p(0x1001), 16, 64, None) == _lib.EZB_ERR_INVALID_ARGUMENT
    assert lib.ezb_attn_decode_paged(fake, fake, fake, fake, fake, fake, 1 << 30, 1, 8, 2, 2, 64, 128, 0, fake, None) == _lib.EZB_ERR_INVALID_ARGUMENT  # no pages
    assert lib.ezb_qwen3_decode_layer(fake, fake, fake, fake, fake, fake, fake, fake, fake, 1 << 30, 1, 128, 2048, 6144,
                                      16, 6, 128, 1e-6, None) == _lib.EZB_ERR_UNSUPPORTED_SHAPE
    assert lib.ezb_qwen3_decode_layer(fake, fake, fake, fake, fake, fake, fake, fake, fake, 1 << 30, 65, 128, 2048, 6144,
                                      16, 8, 128, 1e-6, None) == _lib.EZB_ERR_UNSUPPORTED_SHAPE
    with pytest.raises(ValueError):
        _lib.check(_lib.EZB_ERR_UNSUPPORTED_SHAPE)
    with pytest.raises(_lib.EzbError):
        _lib.check(_lib.EZB_ERR_WORKSPACE)
    assert lib.ezb_qwen3_decode_layer_workspace_bytes(1, 4096, 4096, 12288, 32, 8, 128) > 0
    assert lib.ezb_set_tuning(99, 1) == _lib.EZB_ERR_INVALID_ARGUMENT
    # host-buffer copy: sizes and alignment are checked before any CUDA call
    assert lib.ezb_copy_pinned(None, fake, 64, None) == _lib.EZB_ERR_INVALID_ARGUMENT
    assert lib.ezb_copy_pinned(fake, fake, 24, None) == _lib.EZB_ERR_INVALID_ARGUMENT  # not a multiple of 16
    assert lib.ezb_copy_pinned(fake, odd, 64, None) == _lib.EZB_ERR_INVALID_ARGUMENT
    # the library's all-reduce: buffer, exchange index, size and the ranks' buffers are checked before any launch
    bases = (ctypes.c_void_p * 2)(0x2000, 0x4000)
    assert lib.ezb_tp_allreduce_f32(None, bases, 2, 0, 0, 4, 64, None) == _lib.EZB_ERR_INVALID_ARGUMENT
    assert lib.ezb_tp_allreduce_f32(fake, bases, 2, 0, 2, 4, 64, None) == _lib.EZB_ERR_INVALID_ARGUMENT  # which must be 0 or 1
    assert lib.ezb_tp_allreduce_f32(fake, bases, 2, 0, 0, 1, 6, None) == _lib.EZB_ERR_INVALID_ARGUMENT   # B * H % 4
    assert lib.ezb_tp_allreduce_f32(fake, bases, 2, 2, 0, 4, 64, None) == _lib.EZB_ERR_INVALID_ARGUMENT  # rank outside the world
    assert lib.ezb_tp_allreduce_f32(fake, bases, 9, 0, 0, 4, 64, None) == _lib.EZB_ERR_INVALID_ARGUMENT  # more than 8 ranks


def test_constructor_validation_matches_the_reference_contract():
    with pytest.raises(ValueError, match="power of two"):
        ez.FusedQkNormRopeOp(1, num_heads=16, head_dim=100, max_seq_len=128, position=0)
    with pytest.raises(ValueError, match="position"):
        ez.FusedQkNormRopeOp(1, num_heads=16, head_dim=128, max_seq_len=128, position=128)
    with pytest.raises(ValueError, match="position"):
        ez.FusedQkNormRopeOp(2, num_heads=16, head_dim=128, max_seq_len=128, position=[0, 128])
    with pytest.raises(ValueError, match="divisible"):
        ez.FusedQkNormRopeOp(1, num_heads=16, head_dim=128, max_seq_len=128, position=0, num_kv_heads=6)
    with pytest.raises(ValueError, match="divisible"):
        ez.Qwen3DenseDecodeOp(1, 128, num_heads=16, head_dim=128, hidden_size=2048, intermediate_size=6144, num_kv_heads=6)
    with pytest.raises(ValueError, match="divisible"):
        ez.AttnDecodeOp(1, 16, 128, 128, num_kv_heads=6)
    with pytest.raises(ValueError, match="divisible"):
        ez.FusedOProjFfnOp(1, hidden_size=2048, intermediate_size=6200, num_heads=16, head_dim=128, backend="cuda")
    with pytest.raises(ValueError, match="seq_lens"):
        ez.AttnDecodeOp(2, 8, 128, 128, seq_lens=[1, 129])
    with pytest.raises(KeyError):
        ez.GemvOp(64, 64, backend="triton")


def test_cuda_kernel_classes_refuse_cpu_tensors():
    op = ez.GemvOp(64, 64, backend="cuda")
    with pytest.raises(ValueError, match="CUDA tensor"):
        op(torch.zeros(64, dtype=torch.bfloat16), torch.zeros(64, 64, dtype=torch.bfloat16), torch.zeros(64, dtype=torch.bfloat16))


def test_op_ref_forward_agrees_with_oracle_and_golden_on_cpu():
    """The operators' own torch reference (what backend="ref" runs) is the same
    function as the oracle."""
    g = load_golden("decode_layer_a")
    B, H = g["hidden"].shape
    NH, NKV, D = g["num_heads"], g["num_kv_heads"], g["head_dim"]
    S, I = g["K0"].shape[2], g["Wd"].shape[1]
    op = ez.Qwen3DenseDecodeOp(B, S, H, I, NH, D, backend="ref", num_kv_heads=NKV)
    out = op(g["hidden"], g["K0"].clone(), g["V0"].clone(), g["Wqkv"], g["Wo"], g["Wgu"], g["Wd"])
    assert op.check(out, g["out"])
    assert rel_fro(out, orc.qwen3_dense_decode_ref(g["hidden"], g["K0"].clone(), g["V0"].clone(), g["Wqkv"], g["Wo"],
                                                   g["Wgu"], g["Wd"], NH, NKV, D)) == 0.0

    g = load_golden("o_proj_ffn_a")
    B, Q = g["attn"].shape
    Hh, Ii = g["Wd"].shape
    op = ez.FusedOProjFfnOp(B, Hh, Ii, Q // 32, 32, backend="ref")
    assert op.check(op(*[g[k] for k in ("attn", "residual", "Wo", "post_norm_w", "Wg", "Wu", "Wd")]), g["out"])

    g = load_golden("qk_norm_rope_a")
    B, NQ, D = g["q"].shape
    op = ez.FusedQkNormRopeOp(B, NQ, D, g["cos"].shape[0], g["position"], backend="ref", num_kv_heads=g["k"].shape[1])
    Kc, Vc = g["K0"].clone(), g["V0"].clone()
    out = op(g["q"], g["k"], g["v"], g["qw"], g["kw"], g["cos"], g["sin"], Kc, Vc)
    assert op.check(out, (g["q_out"], g["k_out"])) and torch.equal(Vc, g["V1"])

    g = load_golden("gemv")
    N, K = g["W"].shape
    y = torch.empty(N, dtype=torch.bfloat16)
    op = ez.GemvOp(N, K, backend="ref")
    op(g["x"], g["W"].T.contiguous(), y)
    assert op.check(y, g["y"])

    g = load_golden("attn_decode")
    B, Hq, _, D = g["Q"].shape
    op = ez.AttnDecodeOp(B, Hq, g["K"].shape[2], D, backend="ref", num_kv_heads=g["K"].shape[1])
    assert op.check(op(g["Q"], g["K"], g["V"]), g["out"])


def test_roofline_accounting():
    from ezops_b200.ops.utils.roofline import RooflineResult, algorithmic_bytes_decode_layer, measure_roofline

    a, b = torch.randn(32, 64), torch.randn(64, 128)
    r = measure_roofline(lambda x, y: x @ y, (a, b), {})
    assert r.flops == 2 * 32 * 64 * 128 and r.bytes == a.nbytes + b.nbytes + 32 * 128 * 4
    n = 256
    x, y, z = torch.randn(n), torch.randn(n), torch.empty(n)
    def add_into(p, q, o):
        o.copy_(p + q)

    r = measure_roofline(add_into, (x, y, z), {})
    assert r.flops == n and r.bytes == 3 * n * 4 and abs(r.arithmetic_intensity - 1 / 12) < 1e-12
    assert measure_roofline(lambda v: v + 1, (5,), {}).arithmetic_intensity == float("inf")
    assert RooflineResult(10, 0, 0).arithmetic_intensity == float("inf")
    # Qwen3-8B layer, batch 1, 4096 cached tokens
    assert algorithmic_bytes_decode_layer(1, 4096, 4096, 12288, 32, 128, 8) == 402_653_184
    assert algorithmic_bytes_decode_layer(64, 8192, 5120, 25600, 64, 128, 8) == 3_122_659_328


def test_accuracy_helpers():
    from ezops_b200.ops.utils import bf16_ulp_mismatch, bitwise_equal, check_determinism, check_input_readonly, sqnr_db

    a = torch.tensor([1.0, -2.0, 0.5], dtype=torch.bfloat16)
    b = a.clone()
    b.view(torch.int16)[0] += 1
    assert bf16_ulp_mismatch(a, b) == {0: 2, 1: 1, ">1": 0}
    assert sqnr_db(a, a) == float("inf") and sqnr_db(a, b) > 28.0
    assert not bitwise_equal(torch.tensor([0.0]), torch.tensor([-0.0]))

    def ok(x, out):
        out.copy_(x * 2)

    def bad(x, out):
        x.add_(1)
        out.copy_(x)

    x, out = torch.ones(4), torch.empty(4)
    assert check_determinism(ok, (x,), out) and check_input_readonly(ok, (x,), out)
    assert not check_input_readonly(bad, (x,), out)
