"""The timing protocol ``bench_kernel`` (ezops/ops/utils/bench.py:24-150: eager warm-up with an L2 flush, one call
captured in a CUDA graph with an eager fallback and a warning (:96-109), argument pool (:57-73), median of trial
means) on a real GPU: it returns a positive, repeatable time, every operator of the decode path can be captured, and
a call that cannot be captured is still timed, with the warning."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ez(cuda_device):
    import ezops_b200

    return ezops_b200


def dev(*ts):
    return tuple(t.cuda() for t in ts)


def test_bench_kernel_returns_a_positive_repeatable_time(ez, capsys):
    from ezops_b200.ops.utils import bench_kernel

    n = 1 << 24  # 64 MB per operand: tens of microseconds, far above timer resolution
    op = ez.VectorAddOp(n, backend="cuda")
    a, b, c = torch.randn(n, device="cuda"), torch.randn(n, device="cuda"), torch.empty(n, device="cuda")
    t1 = bench_kernel(op, (a, b, c), n_warmup=5, n_repeat=20, n_trials=3)
    t2 = bench_kernel(op, (a, b, c), n_warmup=5, n_repeat=20, n_trials=3)
    assert t1 > 0 and t2 > 0
    assert 0.7 < t1 / t2 < 1.4, (t1, t2)
    # 3 x 64 MB must take at least what the fastest conceivable HBM allows (10 TB/s) and not seconds
    assert 3 * 4 * n / 10e12 * 1e3 < t1 < 5.0, t1
    assert "capture failed" not in capsys.readouterr().out


def test_every_decode_path_operator_is_captured_not_timed_eagerly(ez, capsys):
    """The reference's benches time a graph replay; a silent eager fallback would add host dispatch to the number.
    All six operators of the path (and the per-row-position form of the q/k-norm + RoPE op) must capture."""
    from ezops_b200 import workloads as wl
    from ezops_b200.ops.utils import bench_kernel

    quick = dict(n_warmup=2, n_repeat=5, n_trials=1)
    times = {}
    x, W, y = dev(*wl.gemv_inputs(1024, 1024))
    times["gemv"] = bench_kernel(ez.GemvOp(1024, 1024, backend="cuda"), (x, W, y), **quick)
    X = torch.randn(32, 4096, device="cuda")
    times["rmsnorm"] = bench_kernel(ez.RmsNormOp(32, 4096, backend="cuda"), (X, torch.empty_like(X)), **quick)
    tensors, positions = wl.qk_norm_rope_inputs(batch=4, num_heads=16, num_kv_heads=8, head_dim=128, max_seq_len=256)
    rope = ez.FusedQkNormRopeOp(4, 16, 128, 256, positions, backend="cuda", num_kv_heads=8)
    times["qk_norm_rope(per-row positions)"] = bench_kernel(rope, dev(*tensors), **quick)
    rope_ref = ez.FusedQkNormRopeOp(4, 16, 128, 256, positions, backend="ref", num_kv_heads=8)
    times["qk_norm_rope ref"] = bench_kernel(rope_ref, dev(*tensors), **quick)
    (Q, K, V), lens = wl.attn_decode_inputs(batch=2, num_heads=16, num_kv_heads=8, head_dim=128, max_len=512, min_len=100)
    attn = ez.AttnDecodeOp(2, 16, 512, 128, backend="cuda", num_kv_heads=8, seq_lens=lens)
    times["attn_decode"] = bench_kernel(attn, dev(Q, K, V), **quick)
    sh = wl.QWEN3_0_6B
    for B in (1, 4):  # batch 1: the single-kernel layer; batch 4: the chained kernels
        data = dev(*wl.decode_layer_inputs(sh, B, 256))
        layer = ez.Qwen3DenseDecodeOp(B, 256, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda", num_kv_heads=sh.num_kv_heads)
        times[f"layer b{B}"] = bench_kernel(layer, data, **quick)
    ffn_in = wl.o_proj_ffn_inputs(sh, 2)
    ffn = ez.FusedOProjFfnOp(2, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda")
    times["o_proj_ffn"] = bench_kernel(ffn, dev(*ffn_in), **quick)
    out = capsys.readouterr().out
    assert "capture failed" not in out, out
    assert all(t > 0 for t in times.values()), times


def test_a_call_that_cannot_be_captured_is_timed_eagerly_with_a_warning(ez, capsys):
    from ezops_b200.ops.utils import bench_kernel

    x = torch.randn(1 << 16, device="cuda")

    def reads_back(t):  # a device-to-host read is illegal inside a stream capture
        return float(t.sum())

    ms = bench_kernel(reads_back, (x,), n_warmup=2, n_repeat=5, n_trials=1)
    out = capsys.readouterr().out
    assert "Warning: CUDA Graph capture failed" in out and "timing eagerly" in out
    assert ms > 0
    # the device is still usable after the failed capture
    torch.cuda.synchronize()
    assert torch.isfinite(x.sum()).item()
