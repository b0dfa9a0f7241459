"""HBM bandwidth calibration: STREAM read / write / copy / triad on the GPU.

Follows the reference's calibrator (benchmarks/hardware/memory/hbm_bandwidth.py:91-171
around hbm_saturation.cu): the triad (a = b + s*c, two reads and one write per
element) over a working set far larger than L2 is the calibration figure; the
other three are printed for context.  The kernels live in the library
(``ezb_hbm_stream``) instead of being compiled at run time.

    python -m benchmarks.hardware.memory.hbm_bandwidth [--size-mb 2048]
"""

from __future__ import annotations

import argparse
import statistics
import sys

from ..gpu_specs import detect_profile, get_specs

OPS = {"read": 0, "write": 1, "copy": 2, "triad": 3}
BYTES_PER_ELEMENT = {"read": 16, "write": 16, "copy": 32, "triad": 48}  # per 128-bit element


def run(profile=None, arch=None, theoretical_bw=None, size_mb=2048, quiet=False, runs=5, reps=50,
        block_sizes=(256, 512, 1024), blocks_per_sm=(2, 4, 8)):
    """Returns ``{gpu_name, arch, profile, measured_gbs, theoretical_gbs, calibration, table}``;
    ``measured_gbs`` is the best triad figure over the launch configurations."""
    import torch

    from ezops_b200 import _lib

    lib = _lib.load()
    props = torch.cuda.get_device_properties(0)
    gpu_name = props.name
    arch = arch or f"sm_{props.major * 10 + props.minor}"
    profile = profile or detect_profile(gpu_name)
    if theoretical_bw is None:
        specs = get_specs(profile) if profile else None
        if not specs:
            raise ValueError("cannot determine the theoretical bandwidth: pass profile or theoretical_bw")
        theoretical_bw = specs["hbm_bw_gb"]

    n_vec4 = size_mb * (1 << 20) // 16
    a, b, c = (torch.empty(n_vec4 * 4, dtype=torch.float32, device="cuda") for _ in range(3))
    b.normal_()
    c.normal_()
    stream = torch.cuda.current_stream().cuda_stream
    table = []
    for name, op in OPS.items():
        for bs in block_sizes:
            for bps in blocks_per_sm:
                def launch():
                    _lib.check(lib.ezb_hbm_stream(op, b.data_ptr(), c.data_ptr(), a.data_ptr(), n_vec4, 0.5, bs, bps, stream))

                for _ in range(5):
                    launch()
                torch.cuda.synchronize()
                times = []
                for _ in range(runs):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(reps):
                        launch()
                    e1.record()
                    torch.cuda.synchronize()
                    times.append(e0.elapsed_time(e1) / reps)
                gbs = [n_vec4 * BYTES_PER_ELEMENT[name] / (t * 1e-3) / 1e9 for t in times]
                table.append({"op": name, "block_size": bs, "blocks_per_sm": bps, "best_gbs": max(gbs),
                              "median_gbs": statistics.median(gbs)})
    measured = max(r["best_gbs"] for r in table if r["op"] == "triad")
    if not quiet:
        print(f"GPU: {gpu_name} | profile: {profile} | working set per array: {size_mb} MB | theoretical {theoretical_bw:.0f} GB/s")
        print("op,block_size,blocks_per_sm,best_gbs,median_gbs,pct_of_theo")
        for r in table:
            print(f"{r['op']},{r['block_size']},{r['blocks_per_sm']},{r['best_gbs']:.1f},{r['median_gbs']:.1f},"
                  f"{100 * r['best_gbs'] / theoretical_bw:.1f}%")
        print(f"triad peak {measured:.1f} GB/s -> calibration {measured / theoretical_bw:.4f}")
    return {"gpu_name": gpu_name, "arch": arch, "profile": profile, "measured_gbs": measured,
            "theoretical_gbs": float(theoretical_bw), "calibration": measured / theoretical_bw, "table": table}


def main():
    ap = argparse.ArgumentParser(description="HBM bandwidth calibration (STREAM kernels)")
    ap.add_argument("--profile", default=None)
    ap.add_argument("--theoretical-bw", type=float, default=None, help="GB/s; overrides the profile table")
    ap.add_argument("--size-mb", type=int, default=2048)
    args = ap.parse_args()
    try:
        run(profile=args.profile, theoretical_bw=args.theoretical_bw, size_mb=args.size_mb)
    except (RuntimeError, ValueError) as exc:
        print(str(exc), file=sys.stderr)
        sys.exit(1)


if __name__ == "__main__":
    main()
