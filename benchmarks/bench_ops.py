#!/usr/bin/env python
"""Per-operator benchmark at the Qwen3 configurations (one GPU).

Follows the reference's bench scripts (benchmarks/bench_gemv.py etc.): for each
workload, run the torch "ref" backend and the "cuda" backend through the
operator API, check the result, time both with ``bench_kernel`` (CUDA graph,
L2 flush before every iteration, median of trial means) and print latency,
achieved GB/s on the algorithmic bytes, the fraction of 8 TB/s and of the
measured copy peak, and the SOL score.  ``--cpu`` adds the same torch reference
timed on the host cores.

    python benchmarks/bench_ops.py [-k gemv,rmsnorm,rope,attn,ffn,layer,stack,pdl_gemm] [--cpu] [--json out.json]

The reference's one-script-per-operator command line (``python benchmarks/bench_gemv.py -h`` / ``-k <backends>``) is
kept by the small ``benchmarks/bench_<op>.py`` files, which run one workload group of this module.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402
from tabulate import tabulate  # noqa: E402

import ezops_b200 as ez  # noqa: E402
from ezops_b200 import workloads as wl  # noqa: E402
from ezops_b200.ops.utils import bench_kernel  # noqa: E402
from ezops_b200.ops.utils.roofline import algorithmic_bytes_attn_decode, algorithmic_bytes_gemv  # noqa: E402

WARMUP, N_REPEAT, N_TRIALS = 10, 50, 3
HBM_NOMINAL_GBS = 8000.0


def measured_hbm_gbs() -> float:
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["hbm_gbs"])
    except Exception:
        return 6650.0


def cpu_time_us(fn, min_calls=3, budget_s=8.0, max_calls=30):
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    fn()
    ts, t_start = [], time.perf_counter()
    while len(ts) < max_calls and (len(ts) < min_calls or time.perf_counter() - t_start < budget_s):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    ts.sort()
    return ts[len(ts) // 2] * 1e6


def dev(*ts):
    return tuple(t.cuda() for t in ts)


def bench(fn, args):
    return bench_kernel(fn, args=args, n_warmup=WARMUP, n_repeat=N_REPEAT, n_trials=N_TRIALS) * 1e3  # us


SOL_HBM_GBS = None  # effective HBM bandwidth of the GPU profile (assets/<profile>.yaml), set in main()


def row(name, us, ref_us, nbytes, ok, cpu_us, peak):
    """``sol_score`` = time at the profile's effective HBM bandwidth / measured time, the
    reference's speed-of-light score for a memory-bound op (benchmarks/bench_gemv.py:62-86)."""
    gbs = nbytes / us / 1e3
    sol_peak = SOL_HBM_GBS or peak
    return {
        "workload": name, "us": us, "torch_ref_us": ref_us, "GB/s": gbs, "frac_8TBs": gbs / HBM_NOMINAL_GBS,
        "frac_measured": gbs / peak, "sol_score": (nbytes / (sol_peak * 1e9)) / (us * 1e-6), "check": ok,
        "cpu_ref_us": cpu_us, "algorithmic_bytes": nbytes,
    }


def run_gemv(cpu, peak):
    x, W, y = wl.gemv_inputs(4096, 4096)
    xd, Wd, yd = dev(x, W, y)
    op = ez.GemvOp(4096, 4096, backend="cuda")
    ref = ez.GemvOp(4096, 4096, backend="ref")
    Wt = Wd.T.contiguous()
    yr = torch.empty_like(yd)
    ref(xd, Wt, yr)
    op(xd, Wd, yd)
    ok = op.check(yd, yr)
    cpu_us = cpu_time_us(lambda: ref._ref_forward(x, W.T.contiguous(), y)) if cpu else None
    return [row("C1 gemv 4096x4096 b1", bench(op, (xd, Wd, yd)), bench(ref, (xd, Wt, yr)), algorithmic_bytes_gemv(4096, 4096), ok, cpu_us, peak)]


def run_rmsnorm(cpu, peak):
    X, w = wl.rmsnorm_inputs(32, 4096)
    Xd, wd = dev(X, w)
    out = torch.empty_like(Xd)
    op = ez.RmsNormOp(32, 4096, backend="cuda", dtype=torch.bfloat16, with_weight=True)
    ref = ez.RmsNormOp(32, 4096, backend="ref", dtype=torch.bfloat16, with_weight=True)
    outr = torch.empty_like(Xd)
    ref(Xd, wd, outr)
    op(Xd, wd, out)
    ok = op.check(out, outr)
    cpu_out = torch.empty_like(X)
    cpu_us = cpu_time_us(lambda: ref._ref_forward(X, w, cpu_out)) if cpu else None
    return [row("C2a rmsnorm bf16+w [32,4096]", bench(op, (Xd, wd, out)), bench(ref, (Xd, wd, outr)), 532480, ok, cpu_us, peak)]


def run_rope(cpu, peak):
    tensors, positions = wl.qk_norm_rope_inputs()
    op = ez.FusedQkNormRopeOp(32, 32, 128, 8192, positions, backend="cuda", num_kv_heads=8)
    ref = ez.FusedQkNormRopeOp(32, 32, 128, 8192, positions, backend="ref", num_kv_heads=8)
    d = dev(*tensors)
    out_r = ref(*[t.clone() for t in d])
    out = op(*[t.clone() for t in d])
    ok = op.check(out, out_r)
    cpu_us = cpu_time_us(lambda: ref._ref_forward(*tensors)) if cpu else None
    return [row("C2b qk-norm+rope+cache 32 tok", bench(op, d), bench(ref, d), 868864, ok, cpu_us, peak)]


def run_attn(cpu, peak):
    (Q, K, V), lens = wl.attn_decode_inputs()
    op = ez.AttnDecodeOp(32, 32, 8192, 128, backend="cuda", num_kv_heads=8, seq_lens=lens)
    ref = ez.AttnDecodeOp(32, 32, 8192, 128, backend="ref", num_kv_heads=8, seq_lens=lens)
    d = dev(Q, K, V)
    out_r, out = ref(*d), op(*d)
    ok = op.check(out, out_r)
    nbytes = algorithmic_bytes_attn_decode(sum(lens), 32, 32, 8, 128)
    cpu_us = cpu_time_us(lambda: ref._ref_forward(Q, K, V)) if cpu else None
    return [row(f"C3 gqa decode b32 sum_len={sum(lens)}", bench(op, d), bench(ref, d), nbytes, ok, cpu_us, peak)]


def run_ffn(cpu, peak):
    sh = wl.QWEN3_8B
    rows = []
    for B in (1, 8):
        args = wl.o_proj_ffn_inputs(sh, B)
        d = dev(*args)
        op = ez.FusedOProjFfnOp(B, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="cuda")
        ref = ez.FusedOProjFfnOp(B, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="ref")
        out_r, out = ref(*d), op(*d)
        nbytes = 2 * (sh.hidden * sh.q_rows + 3 * sh.inter * sh.hidden)
        cpu_us = cpu_time_us(lambda: ref._ref_forward(*args)) if cpu else None
        rows.append(row(f"o_proj+ffn qwen3-8b b{B}", bench(op, d), bench(ref, d), nbytes, op.check(out, out_r), cpu_us, peak))
    return rows


def run_layer(cpu, peak, batches=(1, 8, 32, 64)):
    sh = wl.QWEN3_8B
    rows = []
    for B in batches:
        args = wl.decode_layer_inputs(sh, B, 4096)
        d = dev(*args)
        kw = dict(backend="cuda", num_kv_heads=sh.num_kv_heads)
        op = ez.Qwen3DenseDecodeOp(B, 4096, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, **kw)
        ref = ez.Qwen3DenseDecodeOp(B, 4096, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, backend="ref",
                                    num_kv_heads=sh.num_kv_heads)
        out_r = ref(*[t.clone() for t in d])
        out = op(*[t.clone() for t in d])
        cpu_us = cpu_time_us(lambda: ref._ref_forward(*[t.clone() for t in args]), budget_s=6.0) if cpu else None
        rows.append(row(f"C4 qwen3-8b layer s4096 b{B}", bench(op, d), bench(ref, d), sh.algorithmic_bytes(B, 4096),
                        op.check(out, out_r), cpu_us, peak))
        del d, args
        torch.cuda.empty_cache()
    return rows


def run_stack(cpu, peak, num_layers=36, batches=(1, 8)):
    """All 36 decoder layers of Qwen3-8B in one call (norm weights, RoPE at position S-1): a whole
    decode step apart from the embedding and the LM head.  Inputs are generated on the device
    (14 GB of weights); the check compares with the operator's torch reference on the same GPU."""
    sh, S = wl.QWEN3_8B, 4096
    rows = []
    for B in batches:
        kw = dict(num_kv_heads=sh.num_kv_heads)
        op = ez.Qwen3DecodeStackOp(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, num_layers, backend="cuda", **kw)
        ref = ez.Qwen3DecodeStackOp(B, S, sh.hidden, sh.inter, sh.num_heads, sh.head_dim, num_layers, backend="ref", **kw)
        torch.manual_seed(42)
        hidden, layers, cos, sin = op.gen_data()
        for L in layers:  # the op's default init (fan-in scaling) -> the N(0, 0.02) of the workload definition
            for name in ("Wqkv", "Wo", "Wgu", "Wd"):
                L[name].normal_(0.0, 0.02)
        out_r = ref(hidden, layers, cos, sin)
        out = op(hidden, layers, cos, sin)
        ok = op.check(out, out_r)
        us = bench_kernel(op, args=(hidden, layers, cos, sin), n_warmup=3, n_repeat=10, n_trials=3) * 1e3
        ref_us = bench_kernel(ref, args=(hidden, layers, cos, sin), n_warmup=2, n_repeat=5, n_trials=2) * 1e3
        rows.append(row(f"stack qwen3-8b {num_layers} layers s{S} b{B} (rope, norm w)", us, ref_us,
                        num_layers * sh.algorithmic_bytes(B, S), ok, None, peak))
        del hidden, layers, out, out_r
        torch.cuda.empty_cache()
    return rows


def run_pdl_gemm(cpu, peak):
    """The reference's four chained-GEMM workloads (benchmarks/bench_pdl_gemm.py:36-42): torch, two ordinary launches,
    and the second launch overlapped with the first (programmatic dependent launch).  The interesting number is the
    last column against the one before it."""
    rows = []
    for M, K, N, P, label in ((64, 128, 128, 128, "tiny-mlp"), (64, 512, 512, 512, "small-mlp"), (128, 1024, 1024, 1024, "medium-mlp"),
                              (256, 2048, 2048, 2048, "large-mlp")):
        torch.manual_seed(42)
        ref = ez.PdlGemmOp(M, K, N, P, backend="ref")
        d = ref.gen_data()
        ref(*d)
        want = d[4].clone()
        us = {}
        ok = True
        for backend in ("ref", "cuda", "cuda_pdl"):
            op = ez.PdlGemmOp(M, K, N, P, backend=backend)
            d[4].zero_()
            op(*d)
            ok = ok and op.check(d[4], want)
            us[backend] = bench_kernel(op, args=d, n_warmup=30, n_repeat=200, n_trials=5) * 1e3
        nbytes = 4 * (M * K + K * N + N * P + 2 * M * N + M * P)
        r = row(f"pdl_gemm {label} {M}x{K}x{N}x{P}: no PDL {us['cuda']:.2f} us, PDL", us["cuda_pdl"], us["ref"], nbytes, ok, None, peak)
        r["no_pdl_us"] = us["cuda"]
        rows.append(r)
    return rows


RUNNERS = {"pdl_gemm": run_pdl_gemm, "stack": run_stack, "gemv": run_gemv, "rmsnorm": run_rmsnorm, "rope": run_rope, "attn": run_attn, "ffn": run_ffn, "layer": run_layer}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-k", "--ops", default=",".join(k for k in RUNNERS if k not in ("stack", "pdl_gemm")))
    ap.add_argument("--cpu", action="store_true", help="also time the torch reference on the host cores")
    ap.add_argument("--json", default=None)
    ap.add_argument("--profile", default=None, help="GPU profile under assets/ for the SOL score (default: detected)")
    args = ap.parse_args()
    peak = measured_hbm_gbs()
    from benchmarks.hardware.gpu_specs import detect_profile, load_profile

    global SOL_HBM_GBS
    profile_name = args.profile or detect_profile(torch.cuda.get_device_properties(0).name)
    profile = load_profile(profile_name) if profile_name else None
    if profile and profile.get("hbm", {}).get("effective"):
        SOL_HBM_GBS = profile["hbm"]["effective"] / 1e9
    rows = []
    for name in args.ops.split(","):
        rows += RUNNERS[name.strip()](args.cpu, peak)
    hdr = ["workload", "us", "torch_ref_us", "GB/s", "frac_8TBs", "frac_measured", "sol_score", "check", "cpu_ref_us"]
    fmt = lambda v: f"{v:.3g}" if isinstance(v, float) else v
    print(tabulate([[fmt(r[h]) for h in hdr] for r in rows], headers=hdr, tablefmt="github"))
    print(f"\nprotocol: bench_kernel (CUDA graph, L2 flush per iteration, {N_TRIALS}x{N_REPEAT}); measured HBM copy peak {peak} GB/s; SOL against {SOL_HBM_GBS or peak:.0f} GB/s (profile {profile_name}); "
          f"host threads {len(os.sched_getaffinity(0))}")
    if args.json:
        Path(args.json).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
