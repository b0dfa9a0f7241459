"""The batch-1 decode layer as one persistent kernel (csrc/decode_mega.cu), called through the
operator API and the C ABI entry ``ezb_qwen3_decode_layer``, against the CPU oracle and against
the chained kernels it replaces.

Tolerances: the reference's own acceptance for the layer (relative Frobenius error < 1e-2,
ezops/ops/qwen3_dense_decode.py:64-69); the two GPU paths differ only in the summation order of
the attention phase, so they are held to 5e-3 of each other.  Cache semantics are exact: V slot
S-1 bit-equal to the projected v, every other slot untouched, two calls byte-identical.
"""

import pytest
import torch

from helpers import rel_fro
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


def _shape(name, hidden, inter, heads, kv, d):
    from ezops_b200 import workloads as wl

    return wl.LayerShape(name, hidden, inter, heads, kv, d)


def _run(ez, sh, S, mega: bool):
    from ezops_b200 import _lib
    from ezops_b200 import workloads as wl

    data = wl.decode_layer_inputs(sh, 1, S)
    op = ez.Qwen3DenseDecodeOp(1, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda", num_kv_heads=sh.num_kv_heads)
    dargs = dev(*data)
    launches0 = _lib.load().ezb_launch_count()
    try:
        _lib.set_tuning(mega=1 if mega else 0)
        out = op(*dargs)
        again = op(*dargs)  # on the already-updated cache: idempotent and deterministic
    finally:
        _lib.set_tuning(mega=1)
    launches = (_lib.load().ezb_launch_count() - launches0) // 2
    torch.cuda.synchronize()
    assert torch.equal(out, again)
    return data, dargs, op, out, launches


CASES = [
    # name, hidden, inter, heads, kv heads, head_dim, S
    ("g2", 2048, 6144, 16, 8, 128, 300),        # two query heads per kv head
    ("g2-one-key", 2048, 6144, 16, 8, 128, 1),  # the cache holds only the token being decoded
    ("g2-63", 2048, 6144, 16, 8, 128, 63),
    ("g2-65", 2048, 6144, 16, 8, 128, 65),
    ("g4-8b", 4096, 12288, 32, 8, 128, 4096),   # the headline shape
    ("g4-odd", 4096, 12288, 32, 8, 128, 1001),
    ("g4-long", 4096, 12288, 32, 8, 128, 5003),  # more than one sub-chunk per slice
    ("g8", 2048, 6144, 16, 2, 128, 777),        # eight query heads per kv head, 74 slices per head capped by length
    ("g1", 2048, 2048, 16, 16, 128, 257),
    ("d64", 1024, 3072, 16, 4, 64, 900),        # head_dim 64
    ("small", 1024, 1024, 16, 8, 64, 4000),     # short stages: a slice spans two sub-chunks
]


@pytest.mark.parametrize("name,hidden,inter,heads,kv,d,S", CASES, ids=[c[0] for c in CASES])
def test_single_kernel_layer_vs_oracle_and_chain(ez, name, hidden, inter, heads, kv, d, S):
    sh = _shape(name, hidden, inter, heads, kv, d)
    data, dargs, op, out, launches = _run(ez, sh, S, mega=True)
    assert launches == 1, f"expected the single-kernel path, saw {launches} launches per call"
    hidden_t, K0, V0, Wqkv, Wo, Wgu, Wd = data
    Kr, Vr = K0.clone(), V0.clone()
    ref = orc.qwen3_dense_decode_ref(hidden_t, Kr, Vr, Wqkv, Wo, Wgu, Wd, sh.num_heads, sh.num_kv_heads, sh.head_dim)
    assert op.check(out.cpu(), ref), rel_fro(out, ref)
    Kc, Vc = dargs[1].cpu(), dargs[2].cpu()
    assert torch.allclose(Kc[:, :, -1].float(), Kr[:, :, -1].float(), atol=1e-2, rtol=1e-2)
    assert torch.allclose(Vc[:, :, -1].float(), Vr[:, :, -1].float(), atol=1e-2, rtol=1e-2)
    assert torch.equal(Kc[:, :, :-1], K0[:, :, :-1]) and torch.equal(Vc[:, :, :-1], V0[:, :, :-1])
    for a, t in zip((dargs[0],) + dargs[3:], (hidden_t, Wqkv, Wo, Wgu, Wd)):
        assert torch.equal(a.cpu(), t)  # inputs untouched
    _, dchain, _, chain, chain_launches = _run(ez, sh, S, mega=False)
    assert chain_launches == 5
    assert rel_fro(out, chain) < 5e-3, rel_fro(out, chain)
    assert torch.allclose(dchain[2][:, :, -1].float(), dargs[2][:, :, -1].float(), atol=1e-2, rtol=1e-2)
    assert torch.allclose(dchain[1][:, :, -1].float(), dargs[1][:, :, -1].float(), atol=1e-2, rtol=1e-2)


def test_single_kernel_layer_replayed_from_a_graph(ez):
    """Twenty launches back to back from one CUDA graph, each starting while its predecessor drains: the
    barrier counters must be back at zero every time and every step must give the eager result."""
    from ezops_b200 import _lib
    from ezops_b200 import workloads as wl

    sh, S = wl.QWEN3_VL_2B, 640
    data = wl.decode_layer_inputs(sh, 1, S)
    op = ez.Qwen3DenseDecodeOp(1, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda", num_kv_heads=sh.num_kv_heads)
    k = op._kernel
    dargs = dev(*data)
    bufs = [torch.empty_like(dargs[0]) for _ in range(3)]

    def chain(n):
        x = dargs[0]
        for i in range(n):
            k(x, *dargs[1:], out=bufs[i % 3])
            x = bufs[i % 3]
        return x

    try:
        _lib.set_tuning(pdl_across_calls=1)
        eager = chain(20).clone()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            last = chain(20)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
    finally:
        _lib.set_tuning(pdl_across_calls=0)
    assert torch.isfinite(eager.float()).all()
    assert torch.equal(last, eager)


def test_stack_at_batch_one_uses_the_single_kernel_layer(ez):
    """Norm weights and RoPE inside the single-kernel layer: three layers against the composed oracle."""
    import copy

    from ezops_b200 import _lib
    from ezops_b200 import workloads as wl

    sh, S, NL = wl.QWEN3_VL_2B, 333, 3
    hid, layers, cos, sin = wl.decode_stack_inputs(sh, 1, S, NL)
    ref_layers = copy.deepcopy(layers)
    ref = orc.qwen3_decode_stack_ref(hid, ref_layers, sh.num_heads, sh.num_kv_heads, sh.head_dim, cos, sin)
    op = ez.Qwen3DecodeStackOp(1, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, NL, backend="cuda", num_kv_heads=sh.num_kv_heads)
    dl = [{k: (None if v is None else v.cuda()) for k, v in L.items()} for L in layers]
    n0 = _lib.load().ezb_launch_count()
    got = op(hid.cuda(), dl, cos.cuda(), sin.cuda())
    assert _lib.load().ezb_launch_count() - n0 == NL
    assert rel_fro(got, ref) < 1e-2, rel_fro(got, ref)
    assert torch.allclose(dl[0]["K_cache"][:, :, -1].cpu().float(), ref_layers[0]["K_cache"][:, :, -1].float(), atol=1e-2, rtol=1e-2)
    for L, R in zip(dl, ref_layers):
        assert torch.equal(L["K_cache"][:, :, :-1].cpu(), R["K_cache"][:, :, :-1])
        assert torch.equal(L["V_cache"][:, :, :-1].cpu(), R["V_cache"][:, :, :-1])
