#!/usr/bin/env python
"""Where the time of ONE isolated GEMV launch goes (C1: 4096 x 4096 bf16, batch 1, cold L2).

Prints (1) the floor of the ``bench_kernel`` protocol (a 256-element vector add: event, graph launch of one tiny
kernel, event), (2) the GEMV under the same protocol next to ``torch.mv``, and (3) a device-side timeline of a few
launches, each behind an L2 flush: per CTA the library records %globaltimer when it starts, when its activations
are staged, when its first weight stage has landed and when it exits (``ezb_trace_enable``); the line gives
min / median / max over the CTAs in microseconds since the first CTA started.

    python benchmarks/gemv_isolated_timeline.py [--rows 4096 --cols 4096 --launches 8]
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--launches", type=int, default=8)
    ap.add_argument("--no-protocol", action="store_true",
                    help="skip the bench_kernel measurements: only the few flushed launches of the timeline (what a profiler should see)")
    args = ap.parse_args()

    import ezops_b200 as ez
    from ezops_b200 import _lib, workloads as wl
    from ezops_b200.ops.utils import bench_kernel
    from ezops_b200.ops.utils.bench import l2_flush_buffer

    lib = _lib.load()
    dev = torch.device("cuda")
    N, K = args.rows, args.cols
    x, W, y = (t.cuda() for t in wl.gemv_inputs(N, K))
    op = ez.GemvOp(N, K, backend="cuda")
    tiny = ez.VectorAddOp(256, backend="cuda")
    a, b, c = (torch.randn(256, device=dev) for _ in range(3))
    if not args.no_protocol:
        print(f"protocol floor (vector add, 256 elements): {bench_kernel(tiny, (a, b, c)) * 1e3:.2f} us")
        print(f"GEMV [{N} x {K}] under bench_kernel:        {bench_kernel(op, (x, W, y)) * 1e3:.2f} us")
        print(f"torch.mv under bench_kernel:                {bench_kernel(lambda X, M, Y: torch.mv(M, X, out=Y), (x, W, y)) * 1e3:.2f} us")

    flush = l2_flush_buffer()
    cap = args.launches * 1024 + 64
    rec = torch.zeros(cap * 6, dtype=torch.int64, device=dev)
    cur = torch.zeros(1, dtype=torch.int32, device=dev)
    for _ in range(3):
        flush.zero_()
        op(x, W, y)
    torch.cuda.synchronize()
    lib.ezb_trace_enable(rec.data_ptr(), cur.data_ptr(), cap)
    for _ in range(args.launches):
        flush.zero_()
        op(x, W, y)
        torch.cuda.synchronize()
    lib.ezb_trace_enable(None, None, 0)
    n = int(cur.item())
    r = rec.cpu().numpy().reshape(-1, 6)[:n]
    r = r[np.argsort(r[:, 2])]
    per = n // args.launches
    print(f"{per} CTAs per launch; us since the first CTA of the launch started (min / median / max over CTAs)")
    durations = []
    for L in range(args.launches):
        blk = r[L * per:(L + 1) * per]
        t0 = blk[:, 2].min()

        def stat(col):
            v = (blk[:, col][blk[:, col] > 0] - t0) / 1e3
            return (v.min(), float(np.median(v)), v.max()) if len(v) else (-1.0, -1.0, -1.0)

        durations.append(stat(5)[2])
        print("launch %d: start %5.2f %5.2f %5.2f | staged %5.2f %5.2f %5.2f | first stage landed %5.2f %5.2f %5.2f | exit %5.2f %5.2f %5.2f"
              % ((L,) + stat(2) + stat(3) + stat(4) + stat(5)))
    med = float(np.median(durations))
    print(f"kernel, first start to last exit: median {med:.2f} us = {N * K * 2 / med / 1e3:.0f} GB/s; status {_lib.device_status()}")


if __name__ == "__main__":
    main()
