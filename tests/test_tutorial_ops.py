"""The three teaching operators: reference behaviour on CPU, sm_100a kernels on the GPU.
Shapes and checks follow the reference's tests/test_softmax.py:25-36 (plus its determinism and
read-only-input checks); vector_add and reduce have no tests there and get the same treatment."""

import pytest
import torch

import ezops_b200 as ez
from ezops_b200.ops.utils import check_determinism, check_input_readonly
from oracle import ezops_oracle as orc


def test_reference_forwards_on_cpu():
    torch.manual_seed(0)
    A, B, C = ez.VectorAddOp(1000).gen_data(device="cpu")
    ez.VectorAddOp(1000)(A, B, C)
    assert torch.equal(C, A + B)
    X, Out = ez.SoftmaxOp(3, 100).gen_data(device="cpu")
    ez.SoftmaxOp(3, 100)(X, Out)
    assert torch.allclose(Out.sum(-1), torch.ones(3), atol=1e-6)
    V, S = ez.ReduceOp(5000).gen_data(device="cpu")
    op = ez.ReduceOp(5000)
    op(V, S)
    assert op.check(S, V.double().sum().float().reshape(1)) and op._atol == pytest.approx(5e-4)
    for name in ("vector_add", "softmax", "reduce", "pdl_gemm"):
        assert "cuda" in ez.list_backends(name)
    assert "cuda_pdl" in ez.list_backends("pdl_gemm")
    x, W1, W2, y, z = ez.PdlGemmOp(8, 12, 16, 4).gen_data(device="cpu")
    op = ez.PdlGemmOp(8, 12, 16, 4)
    op(x, W1, W2, y, z)
    y64, z64 = orc.pdl_gemm_ref(x, W1, W2)
    assert op.check(y, y64) and op.check(z, z64)
    with pytest.raises(ValueError, match="divisible by 4"):
        ez.PdlGemmOp(8, 12, 18, 4, backend="cuda")


def test_cpu_oracle_of_the_teaching_ops_agrees_with_the_op_references():
    """The float64 CPU oracle the GPU tests compare against, tied to the operators' own fp32 references."""
    torch.manual_seed(3)
    X = torch.randn(5, 777)
    want = torch.empty_like(X)
    ez.SoftmaxOp(5, 777)(X, want)
    assert torch.allclose(orc.softmax_ref(X), want, atol=1e-6, rtol=1e-5)
    assert torch.allclose(orc.softmax_ref(X).sum(-1), torch.ones(5), atol=1e-6)
    A = torch.randn(10000)
    assert torch.allclose(orc.reduce_sum_ref(A), A.sum().reshape(1), atol=1e-3)
    assert torch.equal(orc.vector_add_ref(A, A), A + A)


@pytest.mark.gpu
@pytest.mark.parametrize("batch,dim", [(1, 64), (128, 1024), (3, 100), (7, 4097), (4096, 4096), (2, 20000),
                                       (3, 12032), (3, 12033), (3, 12288), (3, 12289)])  # around the shared-memory staging limit
def test_softmax_cuda(batch, dim):
    torch.manual_seed(42)
    ref = ez.SoftmaxOp(batch, dim, backend="ref")
    X, _ = ref.gen_data()
    want = orc.softmax_ref(X).cuda()  # CPU oracle, float64 accumulation: independent of this GPU's torch kernels
    op = ez.SoftmaxOp(batch, dim, backend="cuda")
    got = torch.empty_like(want)
    op(X, got)
    assert op.check(got, want), (got - want).abs().max().item()
    assert check_determinism(op, inputs=(X,), outputs=got)
    assert check_input_readonly(op, inputs=(X,), outputs=got)


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 3, 1023, 1 << 20, (1 << 24) + 5])
def test_vector_add_and_reduce_cuda(n):
    torch.manual_seed(1)
    A, B, C = ez.VectorAddOp(n).gen_data()
    op = ez.VectorAddOp(n, backend="cuda")
    op(A, B, C)
    assert torch.equal(C.cpu(), orc.vector_add_ref(A, B))  # CPU oracle
    assert check_input_readonly(op, inputs=(A, B), outputs=C)
    # unaligned views take the scalar path
    if n > 8:
        op1 = ez.VectorAddOp(n - 1, backend="cuda")
        C1 = torch.empty(n, device="cuda")[1:]  # 1-D slices are contiguous but start 4 bytes off the 16-byte grid
        op1(A[1:], B[1:], C1)
        assert torch.equal(C1.cpu(), orc.vector_add_ref(A[1:], B[1:]))
        red1 = ez.ReduceOp(n - 1, backend="cuda")
        out1 = torch.empty(1, device="cuda")
        red1(A[1:], out1)
        assert red1.check(out1.cpu(), orc.reduce_sum_ref(A[1:]))
    red = ez.ReduceOp(n, backend="cuda")
    out = torch.empty(1, device="cuda")
    red(A, out)
    assert red.check(out.cpu(), orc.reduce_sum_ref(A)), (out.item(), A.double().sum().item())
    assert check_determinism(red, inputs=(A,), outputs=out)
    assert check_input_readonly(red, inputs=(A,), outputs=out)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N,P", [(64, 128, 128, 128), (64, 512, 512, 512), (128, 1024, 1024, 1024), (256, 2048, 2048, 2048),
                                     (1, 4, 4, 4), (70, 100, 36, 52), (129, 2052, 68, 200)])
def test_pdl_gemm_cuda(M, K, N, P):
    """The reference's four benchmark workloads (benchmarks/bench_pdl_gemm.py:36-42) and ragged shapes, against the
    float64 CPU oracle with the operator's own acceptance (relative Frobenius error < 1e-2: TF32 inputs); the
    launch with and without programmatic dependent launch must give the same bits."""
    torch.manual_seed(42)
    x, W1, W2, y, z = ez.PdlGemmOp(M, K, N, P).gen_data()
    y64, z64 = orc.pdl_gemm_ref(x, W1, W2)
    plain = ez.PdlGemmOp(M, K, N, P, backend="cuda")
    plain(x, W1, W2, y, z)
    assert plain.check(y.cpu(), y64) and plain.check(z.cpu(), z64)
    rel = ((z.cpu().double() - z64.double()).norm() / z64.double().norm()).item()
    assert rel < 2e-3, rel  # TF32 rounding of two chained products
    pdl = ez.PdlGemmOp(M, K, N, P, backend="cuda_pdl")
    y2, z2 = torch.full_like(y, float("nan")), torch.full_like(z, float("nan"))
    for _ in range(3):
        pdl(x, W1, W2, y2, z2)
    assert torch.equal(y2, y) and torch.equal(z2, z)
    assert check_determinism(pdl, inputs=(x, W1, W2), outputs=(y2, z2))
    assert check_input_readonly(pdl, inputs=(x, W1, W2), outputs=(y2, z2))


@pytest.mark.gpu
def test_pdl_gemm_under_a_cuda_graph():
    torch.manual_seed(1)
    op = ez.PdlGemmOp(64, 512, 512, 512, backend="cuda_pdl")
    x, W1, W2, y, z = op.gen_data()
    op(x, W1, W2, y, z)
    want = z.clone()
    g = torch.cuda.CUDAGraph()
    z.zero_()
    with torch.cuda.graph(g):
        op(x, W1, W2, y, z)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(z, want)
