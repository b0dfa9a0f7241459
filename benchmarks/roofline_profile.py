#!/usr/bin/env python
"""Measure this GPU's roofline ceilings and write its profile YAML.

Same job as the reference's generator (scripts/roofline_profile.py:141-237):
phase 1 is the STREAM-triad HBM calibration, phase 2 the dense matmul peak per
dtype; the file written to ``assets/<profile>.yaml`` holds the spec-sheet
``theoretical`` values and the measured ``calibration`` factors, and
``benchmarks.hardware.gpu_specs.load_profile`` multiplies them.

    python benchmarks/roofline_profile.py [--quick] [--dtypes bf16,fp16] [--output-dir assets]
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from benchmarks.hardware.gpu_specs import detect_profile, get_specs  # noqa: E402

DTYPE_ORDER = ["bf16", "fp16", "tf32", "fp8"]


def _sci(value: float, unit_exp: int) -> str:
    """8000.0, 9 -> '8000e9'; 2250.5, 12 -> '2250.5e12'."""
    return f"{int(value)}e{unit_exp}" if float(value).is_integer() else f"{value:.1f}e{unit_exp}"


def generate_yaml(gpu_name, compute_cap, sm_count, l2_cache_bytes, shared_mem_per_sm, hbm_result, compute_results, specs) -> str:
    """The profile text.  A dtype that was not measured gets the first measured
    calibration as a marked placeholder, as the reference's generator does."""
    out = [
        f"# GPU Profile: {gpu_name}",
        "# Calibration: benchmarks/hardware/ microbenchmarks (STREAM triad, library matmul sweep)",
        "#",
        "# Only theoretical + calibration are stored; effective = theoretical * calibration",
        "# is computed by benchmarks.hardware.gpu_specs.load_profile().",
        "",
        f"gpu: {gpu_name}",
        f"compute_capability: {compute_cap}",
        "",
        f"sm_count: {sm_count}",
    ]
    if l2_cache_bytes is not None:
        out.append(f"l2_cache_size: {l2_cache_bytes}          # {l2_cache_bytes / (1 << 20):.0f} MB")
    if shared_mem_per_sm is not None:
        out.append(f"shared_memory_per_sm: {shared_mem_per_sm}       # {shared_mem_per_sm / 1024:.0f} KB")
    out += ["", "hbm:",
            f"  theoretical: {_sci(hbm_result['theoretical_gbs'], 9)}        # bytes/s, spec sheet",
            f"  calibration: {hbm_result['calibration']:.3f}         # STREAM triad",
            "", "tensor_core:"]
    spec_tf = (specs or {}).get("tensor_core_tflops", {})
    dtypes = [d for d in DTYPE_ORDER if d in spec_tf or d in compute_results]
    dtypes += sorted((set(spec_tf) | set(compute_results)) - set(dtypes))
    placeholder = next((compute_results[d]["calibration"] for d in dtypes
                        if d in compute_results and compute_results[d].get("calibration") is not None), None)
    for d in dtypes:
        r = compute_results.get(d)
        measured = bool(r) and r.get("calibration") is not None
        cal = r["calibration"] if measured else placeholder
        out.append(f"  {d}:")
        if d in spec_tf:
            out.append(f"    theoretical: {_sci(spec_tf[d], 12)}     # FLOPS, spec sheet (dense)")
        if cal is not None:
            out.append(f"    calibration: {cal:.2f}" + ("" if measured else "        # placeholder: not measured"))
        out.append("")
    return "\n".join(out)


def _device_facts():
    import torch

    props = torch.cuda.get_device_properties(0)
    return (props.name, f"{props.major}.{props.minor}", props.multi_processor_count,
            getattr(props, "L2_cache_size", None), getattr(props, "shared_memory_per_multiprocessor", None))


def main():
    ap = argparse.ArgumentParser(description="Generate the GPU roofline profile YAML")
    ap.add_argument("--output-dir", default=str(ROOT / "assets"))
    ap.add_argument("--dtypes", default="bf16,fp16,tf32,fp8")
    ap.add_argument("--quick", action="store_true", help="smaller working set, coarser sweep")
    args = ap.parse_args()

    from benchmarks.hardware.compute.matmul_peak import run as run_matmul
    from benchmarks.hardware.memory.hbm_bandwidth import run as run_hbm

    name, cc, sms, l2, smem = _device_facts()
    profile = detect_profile(name)
    specs = get_specs(profile) if profile else None
    print(f"GPU: {name} | profile: {profile or 'unknown'} | cc {cc} | {sms} SMs")
    if not specs:
        print("this GPU is not in the spec table: no theoretical peaks, nothing to calibrate against", file=sys.stderr)
        sys.exit(1)
    hbm = run_hbm(profile=profile, theoretical_bw=specs["hbm_bw_gb"], size_mb=512 if args.quick else 2048,
                  runs=3 if args.quick else 5, reps=20 if args.quick else 50)
    compute = {}
    for d in [x.strip() for x in args.dtypes.split(",") if x.strip()]:
        try:
            compute[d] = run_matmul(dtype=d, m_step=4096 if args.quick else 1024, n_iter=10 if args.quick else 30)
        except Exception as exc:  # a dtype the library GEMM does not offer here is skipped, not fatal
            print(f"  SKIP {d}: {exc}")
    text = generate_yaml(name, cc, sms, l2, smem, hbm, compute, specs)
    path = Path(args.output_dir) / f"{profile}.yaml"
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(text + "\n")
    print(f"\nsaved {path}\n\n{text}")


if __name__ == "__main__":
    main()
