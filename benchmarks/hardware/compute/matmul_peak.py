"""Dense tensor-core peak through the library GEMM (cuBLAS via torch.matmul).

Counterpart of the reference's matmul sweep
(benchmarks/hardware/compute/matmul_peak.py:163-317): for one dtype, sweep M at
fixed N = K and report the best achieved TFLOP/s; ``calibration`` = best /
spec-sheet dense peak.  This is a calibration of the *roofline ceiling*, the one
place a library GEMM is the right tool.

    python -m benchmarks.hardware.compute.matmul_peak --dtype bf16
"""

from __future__ import annotations

import argparse
import time

from ..gpu_specs import detect_profile, get_specs

DTYPES = ("bf16", "fp16", "tf32", "fp8")


def _time_shape(M, N, K, dtype, n_warmup, n_iter):
    import torch

    if dtype == "fp8":
        f8 = torch.float8_e4m3fn
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16).to(f8)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16).to(f8).t()  # column-major operand
        one = torch.ones((), device="cuda", dtype=torch.float32)
        fn = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    else:
        td = {"bf16": torch.bfloat16, "fp16": torch.float16, "tf32": torch.float32}[dtype]
        a = torch.randn(M, K, device="cuda", dtype=td)
        b = torch.randn(K, N, device="cuda", dtype=td)
        fn = lambda: torch.matmul(a, b)
    for _ in range(n_warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_iter):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return 2.0 * M * N * K * n_iter / (e0.elapsed_time(e1) * 1e-3) / 1e12


def run(dtype="bf16", n=8192, k=8192, m_min=1024, m_max=16384, m_step=1024, warmup=10, n_iter=30,
        gpu_warmup_secs=2, quiet=False, **_ignored):
    """Returns ``{gpu_name, dtype, best_tflops, best_shape, theoretical_tflops, calibration, sweep}``."""
    import torch

    if dtype not in DTYPES:
        raise ValueError(f"dtype must be one of {DTYPES}")
    gpu_name = torch.cuda.get_device_properties(0).name
    profile = detect_profile(gpu_name)
    specs = get_specs(profile) if profile else None
    theo = specs["tensor_core_tflops"].get(dtype) if specs else None
    old_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = dtype == "tf32"
    try:
        t_end = time.time() + gpu_warmup_secs  # bring clocks and power state up
        while time.time() < t_end:
            _time_shape(4096, 4096, 4096, "bf16", 0, 10)
        sweep = []
        for M in range(m_min, m_max + 1, m_step):
            tf = _time_shape(M, n, k, dtype, warmup, n_iter)
            sweep.append((M, tf))
            if not quiet:
                print(f"  {dtype} M={M:6d} N={n} K={k}: {tf:8.1f} TFLOP/s")
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old_tf32
    best_m, best = max(sweep, key=lambda t: t[1])
    return {"gpu_name": gpu_name, "dtype": dtype, "best_tflops": best, "best_shape": (best_m, n, k),
            "theoretical_tflops": theo, "calibration": (best / theo) if theo else None, "sweep": sweep}


def main():
    ap = argparse.ArgumentParser(description="Matmul peak FLOPS finder")
    ap.add_argument("--dtype", default="bf16", choices=DTYPES)
    ap.add_argument("--quick", action="store_true")
    args = ap.parse_args()
    r = run(dtype=args.dtype, m_step=4096 if args.quick else 1024)
    print(f"best {r['best_tflops']:.1f} TFLOP/s at M,N,K={r['best_shape']}; calibration {r['calibration']}")


if __name__ == "__main__":
    main()
