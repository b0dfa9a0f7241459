"""Parity of the sm_100a kernels (called through the operator API, which calls
the C ABI) against the CPU oracle and the golden fixtures.

Tolerances (floating point, bf16 storage):
  * element-wise ops / attention / GEMV: torch.allclose(atol=1e-2, rtol=1e-2),
    the reference's own acceptance (ezops/ops/gemv.py:12-13 etc.);
  * GEMV also: relative error <= 1e-3 against the fp32-accumulated oracle
    rounded to bf16 once;
  * fused layer ops: relative Frobenius error < 1e-2 (the reference's check) and
    max-abs <= 2e-2 on O(1) outputs where that is meaningful for bf16;
  * fp32 RMSNorm: 1e-5.
Integer / copy semantics are exact: V-cache writes bit-equal, every cache slot
other than the written one untouched, two calls byte-identical.
"""

import pytest
import torch

from helpers import frac_within_one_ulp, load_golden, max_abs, rel_fro
from oracle import ezops_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ez(cuda_device):
    import ezops_b200

    return ezops_b200


@pytest.fixture(autouse=True)
def _device_healthy(cuda_device):
    yield
    from ezops_b200 import _lib

    assert _lib.device_status() == 0, "a kernel recorded a device-side fault"


def dev(*ts):
    return tuple(t.cuda() for t in ts)


# ------------------------------------------------------------------ GEMV ---
@pytest.mark.parametrize("N,K", [(192, 320), (100, 64), (1, 16), (4096, 4096), (6144, 4096), (4096, 12288), (5120, 25600)])
def test_gemv_vs_oracle(ez, N, K):
    from ezops_b200 import workloads as wl
    from ezops_b200.ops.utils import check_determinism, check_input_readonly

    x, W, y = wl.gemv_inputs(N, K, seed=7)
    op = ez.GemvOp(N, K, backend="cuda")
    xd, Wd, yd = dev(x, W, y)
    op(xd, Wd, yd)
    ref = orc.gemv_ref(x, W)
    assert op.check(yd.cpu(), ref)
    once = orc.gemv_fp32(x, W).to(torch.bfloat16)
    assert rel_fro(yd, once) <= 1e-3
    assert frac_within_one_ulp(yd, once) > 0.999
    assert check_determinism(op, (xd, Wd), yd)
    assert check_input_readonly(op, (xd, Wd), yd)


def test_gemv_golden(ez):
    g = load_golden("gemv")
    N, K = g["W"].shape
    y = torch.empty(N, dtype=torch.bfloat16, device="cuda")
    ez.GemvOp(N, K, backend="cuda")(g["x"].cuda(), g["W"].cuda(), y)
    assert torch.allclose(y.cpu(), g["y"], atol=1e-2, rtol=1e-2)
    assert rel_fro(y, g["y"]) < 2e-3


def test_gemv_reference_distribution(ez):
    # the reference draws W ~ N(0,1) (ezops/ops/gemv.py:31-33)
    torch.manual_seed(42)
    N = K = 2048
    A, B = torch.randn(K).bfloat16(), torch.randn(N, K).bfloat16()
    C = torch.empty(N, dtype=torch.bfloat16, device="cuda")
    op = ez.GemvOp(N, K, backend="cuda")
    op(A.cuda(), B.cuda(), C)
    assert op.check(C.cpu(), orc.gemv_ref(A, B))


@pytest.mark.parametrize("B,N,K", [(2, 256, 512), (5, 100, 320), (8, 4096, 4096), (8, 512, 12288), (16, 1024, 2048),
                                   (33, 300, 1024), (64, 2048, 4096)])
def test_gemv_batched(ez, B, N, K):
    from ezops_b200 import _lib

    g = torch.Generator().manual_seed(B * 1000 + N)
    X = torch.randn(B, K, generator=g).bfloat16()
    W = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    Y = torch.full((B, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    Xd, Wd = dev(X, W)
    lib = _lib.load()
    ws = torch.zeros(lib.ezb_gemv_workspace_bytes(B, N, K), dtype=torch.uint8, device="cuda")
    _lib.check(lib.ezb_gemv_batched_bf16(Xd.data_ptr(), Wd.data_ptr(), Y.data_ptr(), ws.data_ptr(), ws.numel(), B, N, K,
                                         torch.cuda.current_stream().cuda_stream))
    ref = (X.float() @ W.float().T).to(torch.bfloat16)
    assert rel_fro(Y, ref) <= 1e-3
    assert torch.allclose(Y.cpu().float(), ref.float(), atol=1e-2, rtol=1e-2)


def test_gemv_rejects_bad_k(ez):
    with pytest.raises(ValueError, match="divisible"):
        ez.GemvOp(64, 100, backend="cuda")


# --------------------------------------------------------------- RMSNorm ---
@pytest.mark.parametrize("batch,dim", [(1, 64), (128, 1024), (3, 100), (7, 4097), (4096, 4096), (5, 1025), (2, 20000)])
def test_rmsnorm_f32(ez, batch, dim):
    from ezops_b200.ops.utils import check_determinism, check_input_readonly

    g = torch.Generator().manual_seed(42)
    X = torch.randn(batch, dim, generator=g)
    op = ez.RmsNormOp(batch, dim, backend="cuda")
    Xd = X.cuda()
    Out = torch.empty_like(Xd)
    op(Xd, Out)
    ref = orc.rmsnorm_f32_ref(X)
    assert op.check(Out.cpu(), ref), max_abs(Out, ref)
    assert check_determinism(op, (Xd,), Out)
    assert check_input_readonly(op, (Xd,), Out)


def test_rmsnorm_f32_golden_and_eps(ez):
    g = load_golden("rmsnorm_f32")
    X = g["X"].cuda()
    Out = torch.empty_like(X)
    ez.RmsNormOp(*g["X"].shape, backend="cuda", eps=g["eps"])(X, Out)
    assert torch.allclose(Out.cpu(), g["Out"], atol=1e-5, rtol=1e-5)
    X2 = torch.randn(64, 1024, generator=torch.Generator().manual_seed(1))
    Out2 = torch.empty(64, 1024, device="cuda")
    ez.RmsNormOp(64, 1024, backend="cuda", eps=1e-5)(X2.cuda(), Out2)
    assert torch.allclose(Out2.cpu(), orc.rmsnorm_f32_ref(X2, 1e-5), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("rows,dim,weighted", [(32, 4096, True), (1, 4096, False), (3, 5120, True), (64, 128, True)])
def test_rmsnorm_bf16(ez, rows, dim, weighted):
    from ezops_b200 import workloads as wl

    X, w = wl.rmsnorm_inputs(rows, dim)
    op = ez.RmsNormOp(rows, dim, backend="cuda", dtype=torch.bfloat16, with_weight=weighted)
    Out = torch.empty(rows, dim, dtype=torch.bfloat16, device="cuda")
    if weighted:
        op(X.cuda(), w.cuda(), Out)
    else:
        op(X.cuda(), Out)
    ref = orc.rmsnorm_bf16_ref(X, w if weighted else None)
    assert torch.allclose(Out.cpu().float(), ref.float(), atol=1e-2, rtol=1e-2)
    assert frac_within_one_ulp(Out, ref) > 0.999


# -------------------------------------------------------- QK-norm + RoPE ---
def _run_rope(ez, tensors, position, B, NQ, NKV, D, S):
    q, k, v, qw, kw, cos, sin, K0, V0 = tensors
    Kr, Vr = K0.clone(), V0.clone()
    q_ref, k_ref = orc.qk_norm_rope_ref(q, k, v, qw, kw, cos, sin, Kr, Vr, position)
    op = ez.FusedQkNormRopeOp(B, NQ, D, S, position, backend="cuda", num_kv_heads=NKV)
    args = dev(q, k, v, qw, kw, cos, sin, K0.clone(), V0.clone())
    q_out, k_out = op(*args)
    Kc, Vc = args[7].cpu(), args[8].cpu()
    assert op.check((q_out.cpu(), k_out.cpu()), (q_ref, k_ref))
    assert frac_within_one_ulp(q_out, q_ref) > 0.999 and frac_within_one_ulp(k_out, k_ref) > 0.999
    pos = [position] * B if isinstance(position, int) else position
    for b, p in enumerate(pos):
        assert torch.allclose(Kc[b, :, p].float(), Kr[b, :, p].float(), atol=1e-2, rtol=1e-2)
        assert torch.equal(Kc[b, :, p], k_out[b].cpu())  # cache holds exactly what was returned
        assert torch.equal(Vc[b, :, p], Vr[b, :, p])  # raw copy: bit exact
        mask = torch.ones(S, dtype=torch.bool)
        mask[p] = False
        assert torch.equal(Kc[b][:, mask], K0[b][:, mask]) and torch.equal(Vc[b][:, mask], V0[b][:, mask])
    for a, t in zip(args[:7], tensors[:7]):
        assert torch.equal(a.cpu(), t)  # inputs untouched


@pytest.mark.parametrize("batch,S,position,NKV", [(1, 128, 0, 8), (1, 1024, 512, 8), (2, 1025, 1024, 8), (1, 4096, 1, 4),
                                                  (1, 100, 50, 16), (1, 33, 17, 2)])
def test_qk_norm_rope_reference_cases(ez, batch, S, position, NKV):
    # the cases of the reference's tests/test_fused_qk_norm_rope.py:52-62, with its N(0,1) norm weights
    NQ, D = 16, 128
    g = torch.Generator().manual_seed(42)
    r = lambda *s: torch.randn(*s, generator=g).bfloat16()
    cos, sin = orc.rope_tables(S, D)
    tensors = (r(batch, NQ, D), r(batch, NKV, D), r(batch, NKV, D), r(D), r(D), cos, sin, r(batch, NKV, S, D), r(batch, NKV, S, D))
    _run_rope(ez, tensors, position, batch, NQ, NKV, D, S)


def test_qk_norm_rope_golden(ez):
    for tag in "ab":
        g = load_golden(f"qk_norm_rope_{tag}")
        B, NQ, D = g["q"].shape
        NKV, S = g["k"].shape[1], g["cos"].shape[0]
        op = ez.FusedQkNormRopeOp(B, NQ, D, S, g["position"], backend="cuda", num_kv_heads=NKV)
        Kc, Vc = g["K0"].cuda(), g["V0"].cuda()
        q_out, k_out = op(*dev(g["q"], g["k"], g["v"], g["qw"], g["kw"], g["cos"], g["sin"]), Kc, Vc)
        assert torch.allclose(q_out.cpu().float(), g["q_out"].float(), atol=1e-2, rtol=1e-2)
        assert torch.allclose(k_out.cpu().float(), g["k_out"].float(), atol=1e-2, rtol=1e-2)
        assert torch.equal(Vc.cpu(), g["V1"])
        assert torch.allclose(Kc.cpu().float(), g["K1"].float(), atol=1e-2, rtol=1e-2)


def test_qk_norm_rope_qwen3_8b_per_row_positions(ez):
    from ezops_b200 import workloads as wl

    tensors, positions = wl.qk_norm_rope_inputs(batch=32, max_seq_len=8192)
    _run_rope(ez, tensors, positions, 32, 32, 8, 128, 8192)


def test_qk_norm_rope_constructor_checks(ez):
    with pytest.raises(ValueError, match="power of two"):
        ez.FusedQkNormRopeOp(1, num_heads=16, head_dim=100, max_seq_len=128, position=0, backend="cuda")
    with pytest.raises(ValueError, match="position"):
        ez.FusedQkNormRopeOp(1, num_heads=16, head_dim=128, max_seq_len=128, position=128, backend="cuda")
    with pytest.raises(ValueError, match="divisible"):
        ez.FusedQkNormRopeOp(1, num_heads=16, head_dim=128, max_seq_len=128, position=0, num_kv_heads=6, backend="cuda")


# ------------------------------------------------------------- attention ---
def _attn_case(ez, B, H, NKV, S, D, seq_lens=None, seed=0):
    g = torch.Generator().manual_seed(seed + S)
    r = lambda *s: torch.randn(*s, generator=g).bfloat16()
    Q, K, V = r(B, H, 1, D), r(B, NKV, S, D), r(B, NKV, S, D)
    op = ez.AttnDecodeOp(B, H, S, D, backend="cuda", num_kv_heads=NKV, seq_lens=seq_lens)
    Qd, Kd, Vd = dev(Q, K, V)
    out = op(Qd, Kd, Vd)
    ref = orc.attn_decode_ref(Q, K, V, seq_lens)
    assert out.shape == ref.shape
    assert op.check(out.cpu(), ref), (max_abs(out, ref), rel_fro(out, ref))
    f64 = orc.attn_decode_fp64(Q, K, V, seq_lens)
    assert rel_fro(out, f64) < 6e-3
    out2 = op(Qd, Kd, Vd)
    assert torch.equal(out, out2)  # deterministic
    assert torch.equal(Kd.cpu(), K) and torch.equal(Vd.cpu(), V) and torch.equal(Qd.cpu(), Q)


@pytest.mark.parametrize("B,H,NKV,S,D", [
    (1, 32, 8, 4096, 128), (1, 16, 8, 1000, 128), (2, 16, 8, 1025, 128), (1, 16, 4, 4096, 128), (1, 16, 8, 1, 128),
    (3, 8, 8, 33, 128), (1, 16, 1, 300, 128), (2, 64, 8, 777, 128), (2, 8, 2, 77, 64), (1, 4, 4, 64, 64), (1, 4, 2, 65, 64),
    (4, 32, 8, 8192, 128), (1, 64, 2, 200, 64),
])
def test_attn_decode(ez, B, H, NKV, S, D):
    _attn_case(ez, B, H, NKV, S, D)


def test_attn_decode_golden(ez):
    g = load_golden("attn_decode")
    B, H, _, D = g["Q"].shape
    NKV, S = g["K"].shape[1], g["K"].shape[2]
    out = ez.AttnDecodeOp(B, H, S, D, backend="cuda", num_kv_heads=NKV)(*dev(g["Q"], g["K"], g["V"]))
    assert torch.allclose(out.cpu().float(), g["out"].float(), atol=1e-2, rtol=1e-2)


def test_attn_decode_ragged_lengths(ez):
    _attn_case(ez, 5, 16, 4, 1500, 128, seq_lens=[1, 64, 65, 1499, 1500])
    _attn_case(ez, 3, 8, 2, 300, 64, seq_lens=[7, 300, 129])


def test_attn_decode_qwen3_8b_batch32_ragged(ez):
    from ezops_b200 import workloads as wl

    (Q, K, V), lens = wl.attn_decode_inputs()
    op = ez.AttnDecodeOp(32, 32, 8192, 128, backend="cuda", num_kv_heads=8, seq_lens=lens)
    out = op(*dev(Q, K, V))
    ref = orc.attn_decode_ref(Q, K, V, lens)
    assert op.check(out.cpu(), ref), (max_abs(out, ref), rel_fro(out, ref))
    assert max_abs(out, ref) <= 2e-2


def test_attn_decode_many_small_splits(ez):
    from ezops_b200 import _lib

    old = _lib.get_tuning("attn_min_chunk")
    try:
        _lib.set_tuning(attn_min_chunk=64)
        _attn_case(ez, 1, 16, 8, 1000, 128, seed=5)
        _attn_case(ez, 2, 8, 2, 4096, 128, seq_lens=[100, 4096], seed=6)
    finally:
        _lib.set_tuning(attn_min_chunk=old)


# ----------------------------------------------------------- o_proj + FFN ---
@pytest.mark.parametrize("batch,shape", [(1, "2b"), (1, "0.6b"), (2, "2b"), (4, "2b"), (8, "2b"), (16, "0.6b"), (1, "8b")])
def test_fused_o_proj_ffn(ez, batch, shape):
    from ezops_b200 import workloads as wl

    sh = {"2b": wl.QWEN3_VL_2B, "0.6b": wl.QWEN3_0_6B, "8b": wl.QWEN3_8B}[shape]
    torch.manual_seed(42)
    H, I, Q = sh.hidden, sh.inter, sh.q_rows
    r = lambda *s: torch.randn(*s).bfloat16()
    # the reference's gen_data scaling (ezops/ops/fused_o_proj_ffn.py:96-105)
    args = (r(batch, Q), r(batch, H), r(H, Q) * Q**-0.5, r(H), r(I, H) * H**-0.5, r(I, H) * H**-0.5, r(H, I) * I**-0.5)
    op = ez.FusedOProjFfnOp(batch, H, I, sh.num_heads, sh.head_dim, backend="cuda")
    dargs = dev(*args)
    out = op(*dargs)
    ref = orc.o_proj_ffn_ref(*args)
    assert op.check(out.cpu(), ref), rel_fro(out, ref)
    assert rel_fro(out, orc.o_proj_ffn_fp64(*args)) < 1e-2
    assert torch.equal(op(*dargs), out)
    for a, t in zip(dargs, args):
        assert torch.equal(a.cpu(), t)


def test_fused_o_proj_ffn_golden(ez):
    for tag in "ab":
        g = load_golden(f"o_proj_ffn_{tag}")
        B, Q = g["attn"].shape
        H, I = g["Wd"].shape
        op = ez.FusedOProjFfnOp(B, H, I, Q // 32, 32, backend="cuda")
        out = op(*dev(*[g[k] for k in ("attn", "residual", "Wo", "post_norm_w", "Wg", "Wu", "Wd")]))
        assert rel_fro(out, g["out"]) < 1e-2


def test_fused_o_proj_ffn_divisibility(ez):
    with pytest.raises(ValueError, match="divisible"):
        ez.FusedOProjFfnOp(1, hidden_size=2048, intermediate_size=6200, num_heads=16, head_dim=128, backend="cuda")


# ------------------------------------------------------------ decode layer ---
def _layer_case(ez, batch, seq_len, shape, num_kv_heads=None, std=None, max_abs_bound=None):
    from ezops_b200 import workloads as wl

    sh = shape if num_kv_heads is None else wl.LayerShape(shape.name, shape.hidden, shape.inter, shape.num_heads,
                                                          num_kv_heads, shape.head_dim)
    if std is None:  # the reference's fan-in scaling (ezops/ops/qwen3_dense_decode.py:131-134)
        torch.manual_seed(42)
        r = lambda *s: torch.randn(*s).bfloat16()
        H, I = sh.hidden, sh.inter
        data = (r(batch, H), r(batch, sh.num_kv_heads, seq_len, sh.head_dim), r(batch, sh.num_kv_heads, seq_len, sh.head_dim),
                r(sh.q_rows + 2 * sh.kv_rows, H) * H**-0.5, r(H, sh.q_rows) * sh.q_rows**-0.5, r(2 * I, H) * H**-0.5,
                r(H, I) * I**-0.5)
    else:
        data = wl.decode_layer_inputs(sh, batch, seq_len)
    hidden, K0, V0, Wqkv, Wo, Wgu, Wd = data
    heads = (sh.num_heads, sh.num_kv_heads, sh.head_dim)
    Kr, Vr = K0.clone(), V0.clone()
    ref = orc.qwen3_dense_decode_ref(hidden, Kr, Vr, Wqkv, Wo, Wgu, Wd, *heads)

    op = ez.Qwen3DenseDecodeOp(batch, seq_len, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda",
                               num_kv_heads=sh.num_kv_heads)
    dargs = dev(hidden, K0, V0, Wqkv, Wo, Wgu, Wd)
    out = op(*dargs)
    Kc, Vc = dargs[1].cpu(), dargs[2].cpu()
    assert out.shape == ref.shape
    assert op.check(out.cpu(), ref), rel_fro(out, ref)
    f64 = orc.qwen3_dense_decode_fp64(hidden, K0, V0, Wqkv, Wo, Wgu, Wd, *heads)
    if max_abs_bound is not None:
        # Outputs reach |x| ~ 10, where one bf16 step is 0.0625, so an absolute bound of
        # 2e-2 is only meaningful relative to the output scale: max |diff| <= 2e-2 * max |ref|,
        # and the kernel must be as close to the exact (float64) layer as the reference is.
        assert max_abs(out, ref) <= max_abs_bound * ref.float().abs().max().item(), max_abs(out, ref)
        assert rel_fro(out, f64) <= 1.5 * rel_fro(ref, f64) + 1e-4, (rel_fro(out, f64), rel_fro(ref, f64))
    assert torch.allclose(Kc[:, :, -1].float(), Kr[:, :, -1].float(), atol=1e-2, rtol=1e-2)
    assert torch.allclose(Vc[:, :, -1].float(), Vr[:, :, -1].float(), atol=1e-2, rtol=1e-2)
    assert torch.equal(Kc[:, :, :-1], K0[:, :, :-1]) and torch.equal(Vc[:, :, :-1], V0[:, :, :-1])
    assert rel_fro(out, f64) < 1e-2
    # second call on the already-updated cache: idempotent and deterministic
    out2 = op(*dargs)
    assert torch.equal(out2, out)
    for a, t in zip((dargs[0],) + dargs[3:], (hidden, Wqkv, Wo, Wgu, Wd)):
        assert torch.equal(a.cpu(), t)
    return out, ref


@pytest.mark.parametrize("batch,seq_len,num_kv_heads", [(1, 128, 8), (1, 1000, 8), (2, 1025, 8), (1, 4096, 4), (1, 1, 8)])
def test_decode_layer_reference_cases(ez, batch, seq_len, num_kv_heads):
    from ezops_b200 import workloads as wl

    _layer_case(ez, batch, seq_len, wl.QWEN3_VL_2B, num_kv_heads)


@pytest.mark.parametrize("batch", [1, 8, 32, 64])
def test_decode_layer_qwen3_8b(ez, batch):
    from ezops_b200 import workloads as wl

    _layer_case(ez, batch, 4096, wl.QWEN3_8B, std=0.02, max_abs_bound=2e-2)


def test_decode_layer_qwen3_32b_small_batch(ez):
    from ezops_b200 import workloads as wl

    _layer_case(ez, 2, 512, wl.QWEN3_32B, std=0.02)


def test_decode_layer_qwen3_32b_batch_64_kv_8192(ez):
    """The tensor-parallel configuration of the benchmark on one GPU, unsharded: Qwen3-32B (hidden 5120, 64 q / 8 kv
    heads, intermediate 25600), batch 64, 8192 cached tokens, N(0, 0.02) weights: 0.98 GB of weights and 2.1 GB of KV
    cache.  The oracle computes the attention one kv head at a time (same function as the reference's SDPA call,
    tied to it on a small case in tests/test_oracle_golden.py); acceptance is the reference's relative Frobenius
    bound of 1e-2 (ezops/ops/qwen3_dense_decode.py:64-69)."""
    from ezops_b200 import workloads as wl

    sh, B, S = wl.QWEN3_32B, 64, 8192
    hidden, K0, V0, Wqkv, Wo, Wgu, Wd = wl.decode_layer_inputs(sh, B, S)
    op = ez.Qwen3DenseDecodeOp(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda", num_kv_heads=sh.num_kv_heads)
    dargs = dev(hidden, K0, V0, Wqkv, Wo, Wgu, Wd)
    out = op(*dargs)
    again = op(*dargs)
    torch.cuda.synchronize()
    assert torch.equal(out, again)  # deterministic, idempotent on the updated cache
    # three untouched slots of the caches and the written one, before the oracle overwrites the CPU copies' last slot
    for slot in (0, 4095, S - 2):
        assert torch.equal(dargs[1][:, :, slot].cpu(), K0[:, :, slot]) and torch.equal(dargs[2][:, :, slot].cpu(), V0[:, :, slot])
    ref = orc.qwen3_dense_decode_ref(hidden, K0, V0, Wqkv, Wo, Wgu, Wd, sh.num_heads, sh.num_kv_heads, sh.head_dim, lean_attention=True)
    assert op.check(out.cpu(), ref), rel_fro(out, ref)
    assert rel_fro(out, ref) < 1e-2
    assert max_abs(out, ref) <= 2e-2 * ref.float().abs().max().item() + 0.0626, max_abs(out, ref)  # one bf16 step at |x| ~ 8..16
    assert torch.allclose(dargs[1][:, :, -1].cpu().float(), K0[:, :, -1].float(), atol=1e-2, rtol=1e-2)  # K0 now holds the oracle's new k
    assert torch.allclose(dargs[2][:, :, -1].cpu().float(), V0[:, :, -1].float(), atol=1e-2, rtol=1e-2)


def test_decode_layer_constructor_checks(ez):
    with pytest.raises(ValueError, match="divisible"):
        ez.Qwen3DenseDecodeOp(1, 128, num_heads=16, head_dim=128, hidden_size=2048, intermediate_size=6144,
                              num_kv_heads=6, backend="cuda")
    with pytest.raises(ValueError, match="head_dim"):
        ez.Qwen3DenseDecodeOp(1, 128, num_heads=4, head_dim=32, hidden_size=128, intermediate_size=256, backend="cuda")
    with pytest.raises(ValueError, match="seq_len"):
        ez.Qwen3DenseDecodeOp(1, 0, num_heads=16, head_dim=128, hidden_size=2048, intermediate_size=6144, backend="cuda")


def test_decode_layer_under_cuda_graph(ez):
    from ezops_b200 import workloads as wl

    sh = wl.QWEN3_VL_2B
    data = wl.decode_layer_inputs(sh, 1, 512)
    op = ez.Qwen3DenseDecodeOp(1, 512, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda", num_kv_heads=sh.num_kv_heads)
    dargs = dev(*data)
    eager = op(*dargs)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    static = tuple(t.clone() for t in dargs)
    with torch.cuda.graph(g):
        captured = op(*static)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, eager)


def test_decode_layer_without_pdl_matches(ez):
    from ezops_b200 import _lib
    from ezops_b200 import workloads as wl

    sh = wl.QWEN3_VL_2B
    data = wl.decode_layer_inputs(sh, 2, 300)
    op = ez.Qwen3DenseDecodeOp(2, 300, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda", num_kv_heads=sh.num_kv_heads)
    a = op(*dev(*data))
    try:
        _lib.set_tuning(pdl=0)
        b = op(*dev(*data))
    finally:
        _lib.set_tuning(pdl=1)
    assert torch.equal(a, b)


# ----------------------------------------- tensor-parallel parts on one GPU ---
@pytest.mark.parametrize("tp,batch", [(2, 1), (4, 3), (8, 16)])
def test_tp_parts_sum_to_the_layer(ez, tp, batch):
    """All ranks' local parts run one after the other on this GPU, the two sums
    over ranks done with torch: checks the sharded kernels (fp32 partial
    epilogue, add + norm prologue) without needing several GPUs."""
    from ezops_b200 import tp as tpm
    from ezops_b200 import workloads as wl

    sh = wl.QWEN3_VL_2B if tp < 8 else wl.QWEN3_8B
    S = 700
    hidden, K0, V0, Wqkv, Wo, Wgu, Wd = wl.decode_layer_inputs(sh, batch, S)
    heads = (sh.num_heads, sh.num_kv_heads, sh.head_dim)
    Kr, Vr = K0.clone(), V0.clone()
    ref = orc.qwen3_dense_decode_ref(hidden, Kr, Vr, Wqkv, Wo, Wgu, Wd, *heads)

    hid = hidden.cuda()
    layers, shards, caches = [], [], []
    for r in range(tp):
        lay = tpm.TensorParallelDecodeLayer.__new__(tpm.TensorParallelDecodeLayer)
        lay.group, lay.tp, lay.rank = None, 1, 0  # no process group: sums are done below
        lay.B, lay.S, lay.H, lay.D = batch, S, sh.hidden, sh.head_dim
        lay.NH_l, lay.NKV_l, lay.I_l = sh.num_heads // tp, sh.num_kv_heads // tp, sh.inter // tp
        lay._bufs = None
        layers.append(lay)
        shards.append(dev(*tpm.shard_layer_weights(Wqkv, Wo, Wgu, Wd, *heads, tp, r)))
        caches.append(dev(tpm.shard_kv_cache(K0, tp, r), tpm.shard_kv_cache(V0, tp, r)))
    bufs = [lay._buffers(hid.device) for lay in layers]
    for r, lay in enumerate(layers):
        lay._part_attn(hid, caches[r][0], caches[r][1], shards[r][0], shards[r][1], bufs[r])
    total_o = sum(b["partial_o"] for b in bufs)
    for b in bufs:
        b["partial_o"].copy_(total_o)
    for r, lay in enumerate(layers):
        lay._part_ffn(hid, shards[r][2], shards[r][3], bufs[r])
    total_d = sum(b["partial_d"] for b in bufs)
    out = torch.empty_like(hid)
    bufs[0]["partial_d"].copy_(total_d)
    layers[0]._part_out(out, bufs[0])
    assert rel_fro(out, ref) < 1e-2, rel_fro(out, ref)
    n = sh.num_kv_heads // tp
    for r in range(tp):
        assert torch.allclose(caches[r][0][:, :, -1].cpu().float(), Kr[:, r * n:(r + 1) * n, -1].float(), atol=1e-2, rtol=1e-2)
        assert torch.equal(caches[r][0][:, :, :-1].cpu(), K0[:, r * n:(r + 1) * n, :-1])


@pytest.mark.parametrize("poll_all,pull,strong", [(0, 0, 0), (1, 0, 0), (0, 1, 0), (0, 0, 1)])
@pytest.mark.parametrize("batch", [1, 4, 8, 16, 40])
def test_tp_fused_exchange_world_one_matches_the_layer(ez, batch, poll_all, pull, strong):
    """The fused exchange with one rank pushes into its own inbox: same bits as the
    single-GPU layer, on every one of several calls in a row (the epochs advance)."""
    from ezops_b200 import _lib
    from ezops_b200 import tp as tpm
    from ezops_b200 import workloads as wl

    sh, S = wl.QWEN3_VL_2B, 520
    data = wl.decode_layer_inputs(sh, batch, S)
    op = ez.Qwen3DenseDecodeOp(batch, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda", num_kv_heads=sh.num_kv_heads)
    # batch 1 has two forms of the layer, each with the exchange inside: the single persistent kernel and the chained
    # kernels.  Both are compared with the single-GPU layer of the same form, and they alternate on one set of
    # communication buffers (their epochs and tags must stay compatible).
    forms = (1, 0, 1, 0) if batch == 1 else (1,)
    want = {}
    try:
        for mega in set(forms):
            _lib.set_tuning(mega=mega)
            want[mega] = op(*dev(*data))
    finally:
        _lib.set_tuning(mega=1)
    lay = tpm.TensorParallelDecodeLayer(batch, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, sh.num_kv_heads, exchange="fused")
    try:
        # every form of the exchange, the memory-model-conforming stores (st.relaxed.sys) included
        _lib.set_tuning(tp_poll_all=1 if poll_all else 2, tp_pull=1 if pull else 0, tp_strong_stores=strong)
        for mega in forms:
            _lib.set_tuning(mega=mega)
            for _ in range(3):
                got = lay(*dev(*data))
                assert torch.equal(got, want[mega]), f"mega={mega}"
        assert _lib.device_status() == 0
    finally:
        _lib.set_tuning(tp_poll_all=0, tp_pull=0, tp_strong_stores=0, mega=1)
        torch.cuda.synchronize()
        lay.close()


def test_tp_fused_exchange_rejects_large_batches(ez):
    from ezops_b200 import tp as tpm
    from ezops_b200 import workloads as wl

    sh, S, batch = wl.QWEN3_VL_2B, 300, 65
    data = wl.decode_layer_inputs(sh, batch, S)
    lay = tpm.TensorParallelDecodeLayer(batch, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, sh.num_kv_heads, exchange="fused")
    try:
        with pytest.raises(ValueError):
            lay(*dev(*data))
    finally:
        lay.close()


# ------------------------------------------------- calibration kernels (STREAM) ---
@pytest.mark.parametrize("n_vec4", [1, 1000, 148 * 256 * 4 * 3 + 17])
def test_hbm_stream_kernels_compute_what_they_say(ez, n_vec4):
    from ezops_b200 import _lib

    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(5)
    b = torch.randn(n_vec4 * 4, device="cuda", generator=g)
    c = torch.randn(n_vec4 * 4, device="cuda", generator=g)
    a = torch.zeros(n_vec4 * 4, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.ezb_hbm_stream(3, b.data_ptr(), c.data_ptr(), a.data_ptr(), n_vec4, 0.5, 256, 4, s))
    # the compiler contracts b + s*c into one fma; torch rounds the product first: allow that one rounding
    assert torch.allclose(a, b + 0.5 * c, rtol=0, atol=1e-6)
    _lib.check(lib.ezb_hbm_stream(2, b.data_ptr(), c.data_ptr(), a.data_ptr(), n_vec4, 0.0, 512, 2, s))
    assert torch.equal(a, b)
    _lib.check(lib.ezb_hbm_stream(1, b.data_ptr(), c.data_ptr(), a.data_ptr(), n_vec4, 3.0, 1024, 1, s))
    assert torch.equal(a, torch.full_like(a, 3.0))
    _lib.check(lib.ezb_hbm_stream(0, b.data_ptr(), c.data_ptr(), a.data_ptr(), n_vec4, 0.0, 256, 8, s))
    assert torch.equal(a, torch.full_like(a, 3.0))  # a read pass writes nothing
    with pytest.raises(ValueError):
        _lib.check(lib.ezb_hbm_stream(7, b.data_ptr(), c.data_ptr(), a.data_ptr(), n_vec4, 0.0, 256, 8, s))


# ----------------------------------------------------- multi-layer stack (RoPE, norm weights) ---
def _stack_to_device(layers):
    return [{k: (None if v is None else v.cuda()) for k, v in L.items()} for L in layers]


@pytest.mark.parametrize("batch,num_layers,rope,norm_w", [(1, 3, True, True), (4, 2, True, False), (2, 2, False, True), (16, 2, True, True)])
def test_decode_stack_matches_the_oracle(ez, batch, num_layers, rope, norm_w):
    import copy

    from ezops_b200 import workloads as wl

    sh, S = wl.QWEN3_VL_2B, 333
    hid, layers, cos, sin = wl.decode_stack_inputs(sh, batch, S, num_layers, rope=rope, norm_weights=norm_w)
    ref_layers = copy.deepcopy(layers)
    ref = orc.qwen3_decode_stack_ref(hid, ref_layers, sh.num_heads, sh.num_kv_heads, sh.head_dim, cos, sin)
    op = ez.Qwen3DecodeStackOp(batch, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, num_layers, backend="cuda",
                               num_kv_heads=sh.num_kv_heads, rope=int(rope), norm_weights=int(norm_w))
    dl = _stack_to_device(layers)
    got = op(hid.cuda(), dl, None if cos is None else cos.cuda(), None if sin is None else sin.cuda())
    assert op.check(got.cpu(), ref), rel_fro(got, ref)
    assert rel_fro(got, ref) < 1e-2  # in practice well inside the single-layer bound
    for L, R in zip(dl, ref_layers):
        # first layer's new k is computed from identical inputs; later layers inherit the stream's rounding noise
        assert torch.allclose(L["K_cache"][:, :, -1].cpu().float(), R["K_cache"][:, :, -1].float(), atol=6e-2, rtol=2e-2)
        assert torch.equal(L["K_cache"][:, :, :-1].cpu(), R["K_cache"][:, :, :-1])
        assert torch.equal(L["V_cache"][:, :, :-1].cpu(), R["V_cache"][:, :, :-1])
    assert torch.allclose(dl[0]["K_cache"][:, :, -1].cpu().float(), ref_layers[0]["K_cache"][:, :, -1].float(), atol=1e-2, rtol=1e-2)
    again = op(hid.cuda(), dl, None if cos is None else cos.cuda(), None if sin is None else sin.cuda())
    assert torch.equal(again, got)


def test_decode_stack_of_one_plain_layer_is_the_layer_op(ez):
    from ezops_b200 import workloads as wl

    sh, B, S = wl.QWEN3_VL_2B, 2, 200
    hid, layers, _, _ = wl.decode_stack_inputs(sh, B, S, 1, rope=False, norm_weights=False)
    L = layers[0]
    layer_op = ez.Qwen3DenseDecodeOp(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda", num_kv_heads=sh.num_kv_heads)
    want = layer_op(*dev(hid, L["K_cache"], L["V_cache"], L["Wqkv"], L["Wo"], L["Wgu"], L["Wd"]))
    stack_op = ez.Qwen3DecodeStackOp(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, 1, backend="cuda", num_kv_heads=sh.num_kv_heads)
    got = stack_op(hid.cuda(), _stack_to_device(layers))
    assert torch.equal(got, want)


def test_tp_fused_stack_world_one_matches_the_stack(ez):
    """The tensor-parallel stack with one rank (its exchange pushes into its own inbox, the second
    sum of a layer is gathered by the next layer's QKV kernel) reproduces the single-GPU stack bit for bit."""
    from ezops_b200 import _lib
    from ezops_b200 import tp as tpm
    from ezops_b200 import workloads as wl

    sh, B, S, NL = wl.QWEN3_VL_2B, 2, 260, 3
    hid, layers, cos, sin = wl.decode_stack_inputs(sh, B, S, NL)
    op = ez.Qwen3DecodeStackOp(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, NL, backend="cuda", num_kv_heads=sh.num_kv_heads)
    want = op(hid.cuda(), _stack_to_device(layers), cos.cuda(), sin.cuda())
    stack = tpm.TensorParallelDecodeStack(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, sh.num_kv_heads, NL)
    try:
        dl = _stack_to_device(layers)
        for _ in range(2):
            got = stack(hid.cuda(), dl, cos.cuda(), sin.cuda())
            assert torch.equal(got, want)
        assert _lib.device_status() == 0
    finally:
        torch.cuda.synchronize()
        stack.close()



@pytest.mark.parametrize("batch,lens", [(4, [333, 17, 128, 65]), (1, [200]), (16, [333, 1, 64, 65, 129, 300, 2, 77, 333, 200, 100, 50, 25, 12, 6, 3])])
def test_decode_stack_with_per_row_lengths(ez, batch, lens):
    """Rows of different lengths in one batch: the new token of row b goes to slot lens[b]-1, the row
    attends to its own prefix and RoPE uses that slot's table row; everything else in the caches stays."""
    import copy

    from ezops_b200 import workloads as wl

    sh, S, NL = wl.QWEN3_VL_2B, 333, 2
    hid, layers, cos, sin = wl.decode_stack_inputs(sh, batch, S, NL)
    ref_layers = copy.deepcopy(layers)
    ref = orc.qwen3_decode_stack_ref(hid, ref_layers, sh.num_heads, sh.num_kv_heads, sh.head_dim, cos, sin, seq_lens=lens)
    op = ez.Qwen3DecodeStackOp(batch, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, NL, backend="cuda",
                               num_kv_heads=sh.num_kv_heads, seq_lens=lens)
    dl = _stack_to_device(layers)
    got = op(hid.cuda(), dl, cos.cuda(), sin.cuda())
    assert rel_fro(got, ref) < 1e-2, rel_fro(got, ref)
    for L, R, L0 in zip(dl, ref_layers, layers):
        for b, n in enumerate(lens):
            keep = [i for i in range(S) if i != n - 1]
            assert torch.equal(L["K_cache"][b][:, keep].cpu(), L0["K_cache"][b][:, keep])
            assert torch.equal(L["V_cache"][b][:, keep].cpu(), L0["V_cache"][b][:, keep])
            assert torch.allclose(L["K_cache"][b][:, n - 1].cpu().float(), R["K_cache"][b][:, n - 1].float(), atol=6e-2, rtol=2e-2)
    again = op(hid.cuda(), dl, cos.cuda(), sin.cuda())
    assert torch.equal(again, got)


# ------------------------------------------------------------------ paged KV caches ---
def _to_pages(cache, page_size, perm, extra_pages=3):
    """Contiguous cache [B, NKV, S, D] -> (pool [pages, NKV, P, D], page_table [B, S/P]) with shuffled page ids."""
    B, NKV, S, D = cache.shape
    n = S // page_size
    pool = torch.randn(B * n + extra_pages, NKV, page_size, D, dtype=cache.dtype)  # unmapped pages hold noise
    table = perm[: B * n].view(B, n).to(torch.int32)
    for b in range(B):
        for i in range(n):
            pool[table[b, i]] = cache[b, :, i * page_size:(i + 1) * page_size]
    return pool, table


def _from_pages(pool, table, page_size):
    B, n = table.shape
    return torch.stack([torch.cat([pool[table[b, i]] for i in range(n)], dim=1) for b in range(B)])


@pytest.mark.parametrize("page_size", [64, 256])
def test_paged_attention_matches_contiguous(ez, page_size):
    from ezops_b200 import workloads as wl

    B, H, NKV, D, S = 5, 16, 4, 128, 1024
    (Q, K, V), _ = wl.attn_decode_inputs(batch=B, num_heads=H, num_kv_heads=NKV, head_dim=D, max_len=S, min_len=1)
    lens = [1024, 1, 65, 700, 256]
    perm = torch.randperm(B * (S // page_size) + 3, generator=torch.Generator().manual_seed(3))
    Kp, table = _to_pages(K, page_size, perm)
    Vp, _ = _to_pages(V, page_size, perm)
    op = ez.AttnDecodeOp(B, H, S, D, backend="cuda", num_kv_heads=NKV, seq_lens=lens)
    want = op(*dev(Q, K, V))
    lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
    got = op._kernel.call_paged(Q.cuda(), Kp.cuda(), Vp.cuda(), table.cuda(), lens_d, page_size)
    assert torch.equal(got, want)  # same kernel, same tiles, only the addresses differ
    assert torch.allclose(got.cpu().float(), orc.attn_decode_ref(Q, K, V, seq_lens=lens).float(), atol=1e-2, rtol=1e-2)


def test_paged_decode_stack_matches_the_contiguous_stack(ez):
    import copy

    from ezops_b200 import workloads as wl

    sh, B, S, NL, P = wl.QWEN3_VL_2B, 3, 512, 2, 128
    lens = [512, 130, 7]
    hid, layers, cos, sin = wl.decode_stack_inputs(sh, B, S, NL)
    ref_layers = copy.deepcopy(layers)
    ref = orc.qwen3_decode_stack_ref(hid, ref_layers, sh.num_heads, sh.num_kv_heads, sh.head_dim, cos, sin, seq_lens=lens)
    perm = torch.randperm(B * (S // P) + 3, generator=torch.Generator().manual_seed(5))
    paged, table = [], None
    for L in layers:
        Kp, table = _to_pages(L["K_cache"], P, perm)
        Vp, _ = _to_pages(L["V_cache"], P, perm)
        paged.append({**L, "K_cache": Kp, "V_cache": Vp})
    op = ez.Qwen3DecodeStackOp(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, NL, backend="cuda", num_kv_heads=sh.num_kv_heads)
    dl = _stack_to_device(paged)
    lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
    got = op._kernel(hid.cuda(), dl, cos.cuda(), sin.cuda(), seq_lens=lens_d, page_table=table.cuda(), page_size=P)
    assert rel_fro(got, ref) < 1e-2, rel_fro(got, ref)
    contiguous = ez.Qwen3DecodeStackOp(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, NL, backend="cuda",
                                       num_kv_heads=sh.num_kv_heads, seq_lens=lens)
    cl = _stack_to_device(layers)
    assert torch.equal(got, contiguous(hid.cuda(), cl, cos.cuda(), sin.cuda()))
    for Lp, Lc in zip(dl, cl):  # the new tokens landed in the right pages, nothing else moved
        assert torch.equal(_from_pages(Lp["K_cache"].cpu(), table, P), Lc["K_cache"].cpu())
        assert torch.equal(_from_pages(Lp["V_cache"].cpu(), table, P), Lc["V_cache"].cpu())



def test_paged_attention_reports_a_page_id_outside_the_pool(ez):
    """A stale or unallocated (-1) page-table entry inside a row's valid length must not be dereferenced: the call
    returns, the status word reads 0x302, rows with good tables are still right, and the next call is healthy."""
    from ezops_b200 import _lib
    from ezops_b200 import workloads as wl

    B, H, NKV, D, S, P = 3, 16, 4, 128, 512, 64
    (Q, K, V), _ = wl.attn_decode_inputs(batch=B, num_heads=H, num_kv_heads=NKV, head_dim=D, max_len=S, min_len=1)
    lens = [512, 300, 129]
    perm = torch.randperm(B * (S // P) + 3, generator=torch.Generator().manual_seed(9))
    Kp, table = _to_pages(K, P, perm)
    Vp, _ = _to_pages(V, P, perm)
    bad = table.clone()
    bad[1, 2] = -1                 # inside row 1's 300 keys: "unallocated"
    bad[2, 1] = Kp.shape[0] + 5    # inside row 2's 129 keys: beyond the pool
    bad[2, 7] = -1                 # beyond row 2's length: never looked at
    op = ez.AttnDecodeOp(B, H, S, D, backend="cuda", num_kv_heads=NKV, seq_lens=lens)
    lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
    got = op._kernel.call_paged(Q.cuda(), Kp.cuda(), Vp.cuda(), bad.cuda(), lens_d, P)
    assert _lib.device_status() == 0x302  # reads and clears
    ref = orc.attn_decode_ref(Q, K, V, seq_lens=lens)
    assert torch.allclose(got[0].cpu().float(), ref[0].float(), atol=1e-2, rtol=1e-2)  # the row with a good table
    again = op._kernel.call_paged(Q.cuda(), Kp.cuda(), Vp.cuda(), table.cuda(), lens_d, P)
    assert _lib.device_status() == 0
    assert torch.allclose(again.cpu().float(), ref.float(), atol=1e-2, rtol=1e-2)


def test_fused_exchange_wait_runs_out_and_poisons_the_chain(ez):
    """A peer that never delivers: world of two with both communication buffers on this GPU and nobody playing
    rank 1.  With the wait budget at 2 ms the gathering kernel gives up, records 0x201, stores nothing and pushes
    nothing; the kernels behind it see the fault and stay silent too, so the output buffer is untouched.  Nothing
    traps, nothing is left spinning, and after clearing the status word a world-of-one call is healthy again."""
    import ctypes

    from ezops_b200 import _lib
    from ezops_b200 import workloads as wl

    lib = _lib.load()
    sh, B, S = wl.QWEN3_0_6B, 1, 200
    data = dev(*wl.decode_layer_inputs(sh, B, S))
    hidden, Kc, Vc, Wqkv, Wo, Wgu, Wd = data
    K0 = Kc.clone()
    nbytes = lib.ezb_tp_comm_bytes(B, sh.hidden)
    bufs = [ctypes.c_void_p(), ctypes.c_void_p()]
    for b in bufs:
        _lib.check(lib.ezb_tp_comm_alloc(nbytes, ctypes.byref(b)))
    ws = torch.zeros(lib.ezb_qwen3_decode_layer_workspace_bytes(B, S, sh.hidden, sh.inter, sh.num_heads, sh.num_kv_heads, sh.head_dim),
                     dtype=torch.uint8, device="cuda")
    out = torch.full_like(hidden, 7.0)
    s = torch.cuda.current_stream().cuda_stream

    def call(world):
        bases = (ctypes.c_void_p * world)(*[b.value for b in bufs[:world]])
        return lib.ezb_qwen3_decode_layer_tp_fused(
            hidden.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), Wqkv.data_ptr(), Wo.data_ptr(), Wgu.data_ptr(), Wd.data_ptr(),
            out.data_ptr(), ws.data_ptr(), ws.numel(), bases, world, 0, B, S, sh.hidden, sh.inter, sh.num_heads,
            sh.num_kv_heads, sh.head_dim, 1e-6, s)

    try:
        _lib.set_tuning(tp_wait_limit_ms=2)
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        assert call(2) == _lib.EZB_OK  # the call only enqueues; the fault is found on the device
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 500.0  # gave up after about the budget, not after seconds
        word = ctypes.c_uint(0)
        assert lib.ezb_device_status(ctypes.byref(word), 0) == _lib.EZB_ERR_DEVICE_FAULT and word.value == 0x201
        assert torch.equal(out, torch.full_like(out, 7.0)), "a rank that gave up must not publish a result"
        # a second call while the fault stands: still silent (no gather, no push), and quick
        t0.record()
        assert call(2) == _lib.EZB_OK
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 50.0
        assert torch.equal(out, torch.full_like(out, 7.0))
        assert _lib.device_status() == 0x201  # reads and clears
    finally:
        _lib.set_tuning(tp_wait_limit_ms=5000)
        torch.cuda.synchronize()
        _lib.device_status()
    # fresh buffers (the aborted calls left epochs and cells in an undefined state), world of one: healthy again
    for b in bufs:
        _lib.check(lib.ezb_tp_comm_free(b))
    bufs = [ctypes.c_void_p()]
    _lib.check(lib.ezb_tp_comm_alloc(nbytes, ctypes.byref(bufs[0])))
    try:
        Kc.copy_(K0)
        assert call(1) == _lib.EZB_OK
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        ref = orc.qwen3_dense_decode_ref(*(t.cpu() for t in (hidden, K0, Vc, Wqkv, Wo, Wgu, Wd)), sh.num_heads, sh.num_kv_heads, sh.head_dim)
        assert rel_fro(out, ref) < 1e-2
    finally:
        torch.cuda.synchronize()
        _lib.check(lib.ezb_tp_comm_free(bufs[0]))


# ------------------------------------------------ host buffers at the boundary ---
@pytest.mark.parametrize("direct", [True, False])
@pytest.mark.parametrize("batch", [1, 5])
def test_layer_takes_pinned_host_buffers(ez, batch, direct):
    """A host application holds the step's input and result in pinned host memory: the operator copies in, runs
    the layer and copies out as one chain on the stream (ezb_copy_pinned); the result equals the device call bit for
    bit, also when the three calls are replayed from a CUDA graph, and pageable memory is refused."""
    from ezops_b200 import _lib
    from ezops_b200 import workloads as wl

    sh, S = wl.QWEN3_0_6B, 300
    data = wl.decode_layer_inputs(sh, batch, S)
    hidden, rest = data[0], dev(*data[1:])
    op = ez.Qwen3DenseDecodeOp(batch, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda", num_kv_heads=sh.num_kv_heads)
    op._kernel.direct_host_output = direct  # the last kernel stores into the host buffer | a copy-out kernel does
    want = op(hidden.cuda(), *rest).cpu()
    h_in, h_out = hidden.clone().pin_memory(), torch.zeros_like(hidden).pin_memory()
    got = op._kernel(h_in, *rest, out=h_out)
    torch.cuda.synchronize()
    assert got is h_out and torch.equal(h_out, want)
    # the same three calls from a graph, with a new input written by the host between replays
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            op._kernel(h_in, *rest, out=h_out)
    for scale in (0.5, 2.0):
        h_in.copy_((hidden.float() * scale).to(torch.bfloat16))
        want = op(h_in.cuda(), *rest).cpu()
        h_out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(h_out, want)
    # pageable host memory has no device address: refused, nothing launched
    lib = _lib.load()
    pageable = torch.zeros(batch, sh.hidden, dtype=torch.bfloat16)
    rc = lib.ezb_copy_pinned(rest[0].data_ptr(), pageable.data_ptr(), pageable.numel() * 2, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.EZB_ERR_INVALID_ARGUMENT
    assert b"pinned" in lib.ezb_last_error_message()
    with pytest.raises(ValueError, match="pinned"):
        op._kernel(pageable, *rest)


@pytest.mark.parametrize("batch", [1, 4, 16, 40])
def test_tp_peer_allreduce_world_one_matches_the_three_part_form(ez, batch):
    """The library's own sum over ranks (ezb_tp_allreduce_f32) with one rank: the partial goes through the
    communication buffer and comes back unchanged, so the layer equals the three-part form bit for bit, call after
    call (the flags' epochs advance) and from a CUDA graph."""
    from ezops_b200 import _lib
    from ezops_b200 import tp as tpm
    from ezops_b200 import workloads as wl

    sh, S = wl.QWEN3_VL_2B, 333
    data = dev(*wl.decode_layer_inputs(sh, batch, S))
    args = (batch, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, sh.num_kv_heads)
    want = tpm.TensorParallelDecodeLayer(*args)(*data)
    lay = tpm.TensorParallelDecodeLayer(*args, exchange="peer")
    try:
        for _ in range(3):
            assert torch.equal(lay(*data), want)
        out = torch.empty_like(want)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                lay(*data, out=out)
        for _ in range(3):
            out.zero_()
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, want)
        assert _lib.device_status() == 0
    finally:
        torch.cuda.synchronize()
        lay.close()


def test_peer_allreduce_wait_runs_out_and_leaves_the_buffer_alone(ez):
    """The library's all-reduce with a peer that never delivers (a world of two, both communication buffers on this
    GPU, nobody playing rank 1, budget 2 ms): the kernel returns, the status word reads 0x201, the buffer still
    holds the rank's own partial, a second call while the fault stands returns at once, and after clearing the word
    a world-of-one call is healthy (the sum of one rank is the partial itself)."""
    import ctypes

    from ezops_b200 import _lib

    lib = _lib.load()
    B, H = 16, 2048
    nbytes = lib.ezb_tp_comm_bytes(B, H)
    bufs = [ctypes.c_void_p(), ctypes.c_void_p()]
    for b in bufs:
        _lib.check(lib.ezb_tp_comm_alloc(nbytes, ctypes.byref(b)))
    part = torch.randn(B, H, device="cuda")
    keep = part.clone()
    s = torch.cuda.current_stream().cuda_stream

    def call(world, which):
        bases = (ctypes.c_void_p * world)(*[b.value for b in bufs[:world]])
        return lib.ezb_tp_allreduce_f32(part.data_ptr(), bases, world, 0, which, B, H, s)

    try:
        _lib.set_tuning(tp_wait_limit_ms=2)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        assert call(2, 0) == _lib.EZB_OK  # the call only enqueues; the fault is found on the device
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 500.0
        word = ctypes.c_uint(0)
        assert lib.ezb_device_status(ctypes.byref(word), 0) == _lib.EZB_ERR_DEVICE_FAULT and word.value == 0x201
        assert torch.equal(part, keep), "a rank that gave up must not publish a sum"
        t0.record()
        assert call(2, 1) == _lib.EZB_OK  # poisoned: returns at once
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 50.0 and torch.equal(part, keep)
        assert _lib.device_status() == 0x201  # reads and clears
    finally:
        _lib.set_tuning(tp_wait_limit_ms=5000)
        torch.cuda.synchronize()
        _lib.device_status()
        for b in bufs:
            _lib.check(lib.ezb_tp_comm_free(b))
    one = ctypes.c_void_p()
    _lib.check(lib.ezb_tp_comm_alloc(nbytes, ctypes.byref(one)))
    bufs = [one]
    try:
        for which in (0, 1, 0):
            assert call(1, which) == _lib.EZB_OK
        torch.cuda.synchronize()
        assert _lib.device_status() == 0 and torch.equal(part, keep)
    finally:
        torch.cuda.synchronize()
        _lib.check(lib.ezb_tp_comm_free(one))
