"""The three teaching operators: reference behaviour on CPU, sm_100a kernels on the GPU.
Shapes and checks follow the reference's tests/test_softmax.py:25-36 (plus its determinism and
read-only-input checks); vector_add and reduce have no tests there and get the same treatment."""

import pytest
import torch

import ezops_b200 as ez
from ezops_b200.ops.utils import check_determinism, check_input_readonly


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
    for name in ("vector_add", "softmax", "reduce"):
        assert "cuda" in ez.list_backends(name)


@pytest.mark.gpu
@pytest.mark.parametrize("batch,dim", [(1, 64), (128, 1024), (3, 100), (7, 4097), (4096, 4096), (2, 20000)])
def test_softmax_cuda(batch, dim):
    torch.manual_seed(42)
    ref = ez.SoftmaxOp(batch, dim, backend="ref")
    X, want = ref.gen_data()
    ref._ref_forward(X, want)
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
    assert torch.equal(C, A + B)
    assert check_input_readonly(op, inputs=(A, B), outputs=C)
    # unaligned views take the scalar path
    if n > 8:
        op1 = ez.VectorAddOp(n - 1, backend="cuda")
        C1 = torch.empty(n, device="cuda")[1:]  # 1-D slices are contiguous but start 4 bytes off the 16-byte grid
        op1(A[1:], B[1:], C1)
        assert torch.equal(C1, A[1:] + B[1:])
        red1 = ez.ReduceOp(n - 1, backend="cuda")
        out1 = torch.empty(1, device="cuda")
        red1(A[1:], out1)
        assert red1.check(out1, A[1:].double().sum().float().reshape(1))
    red = ez.ReduceOp(n, backend="cuda")
    out = torch.empty(1, device="cuda")
    red(A, out)
    assert red.check(out, A.double().sum().float().reshape(1)), (out.item(), A.double().sum().item())
    assert check_determinism(red, inputs=(A,), outputs=out)
    assert check_input_readonly(red, inputs=(A,), outputs=out)
