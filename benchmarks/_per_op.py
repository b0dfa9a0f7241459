"""Command line of the reference's per-operator benchmark scripts (benchmarks/bench_gemv.py:177-212 and its
siblings): ``-h`` lists the registered backends of the operator and exits, ``-k a,b`` selects backends (the torch
reference is always timed beside them).  The measurement itself is one workload group of ``benchmarks/bench_ops.py``
(bench_kernel protocol, SOL score against the GPU profile)."""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def main(op_name: str, group: str, description: str) -> None:
    import ezops_b200 as ez

    backends = ez.list_backends(op_name)
    ap = argparse.ArgumentParser(add_help=False, description=description)
    ap.add_argument("-h", action="store_true", dest="list_backends", help="List available backends and exit")
    ap.add_argument("-k", "--backends", type=str, default=None,
                    help="Comma-separated list of backends to benchmark (ref is always included)")
    ap.add_argument("--cpu", action="store_true", help="also time the torch reference on the host cores")
    args = ap.parse_args()
    if args.list_backends:
        print("Available backends:", ", ".join(backends))
        return
    if args.backends is not None:
        selected = [b.strip() for b in args.backends.split(",")]
        invalid = [b for b in selected if b != "ref" and b not in backends]
        if invalid:
            print(f"Unknown backends: {', '.join(invalid)}")
            print(f"Available: {', '.join(backends)}")
            return
        if not [b for b in selected if b != "ref"]:
            print("Nothing to compare: name at least one backend besides ref")
            return
    from benchmarks import bench_ops

    sys.argv = [sys.argv[0], "-k", group] + (["--cpu"] if args.cpu else [])
    bench_ops.main()
