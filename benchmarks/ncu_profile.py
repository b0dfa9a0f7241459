#!/usr/bin/env python
"""Profile one operator's kernels with Nsight Compute.

Command-line behaviour of the reference's tool (scripts/ncu_profile.py:180-294):
``<op_name>`` in snake case, ``-k`` backends (``ref`` = the op's torch
reference; ``all`` = every registered backend), ``-p`` constructor parameters
(``N=4096,K=4096`` or positional ``4096,4096``), ``-o`` output directory, ``-w``
warm-up iterations; ``-h`` alone lists the ops, ``<op> -h`` its backends and
parameters.  For every backend it warms the kernel up in this process, writes a
three-line driver script and runs it under ``ncu --set full``.

Differences, all about sharing a GPU safely: the driver script is first run
WITHOUT ncu and must exit 0 before it is profiled; ncu always gets
``--clock-control none`` (it would otherwise lock the clocks for the next user);
``-c`` bounds the captured launches (default 3) and ``-K`` restricts the capture
to kernels whose name matches a regex.

    python benchmarks/ncu_profile.py gemv -k cuda -p N=4096,K=4096
"""

from __future__ import annotations

import argparse
import importlib
import shutil
import subprocess
import sys
import textwrap
from datetime import datetime
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
PACKAGE = "ezops_b200"


def op_name_to_class(op_name: str) -> str:
    """'fused_qk_norm_rope' -> 'FusedQkNormRopeOp' (the reference's rule).  Where the package
    spells the class differently ('rmsnorm' is RmsNormOp), the exported class whose name
    matches without regard to case wins, so every registered op can be profiled."""
    guess = "".join(part.capitalize() for part in op_name.split("_")) + "Op"
    try:
        mod = importlib.import_module(PACKAGE)
    except ImportError:
        return guess
    if hasattr(mod, guess):
        return guess
    for name in dir(mod):
        if name.lower() == guess.lower():
            return name
    return guess


def parse_params(text: str) -> tuple[list, dict]:
    """'M=5,N=10' -> ([], {'M': 5, 'N': 10}); '5,10,1e-6' -> ([5, 10, 1e-06], {})."""
    def number(v: str):
        v = v.strip()
        try:
            return int(v)
        except ValueError:
            return float(v)

    if not text:
        return [], {}
    if "=" in text:
        return [], {k.strip(): number(v) for k, v in (pair.split("=") for pair in text.split(","))}
    return [number(v) for v in text.split(",")], {}


def _ctor_args(pos: list, kw: dict, backend: str | None) -> str:
    parts = [repr(a) for a in pos] + [f"{k}={v!r}" for k, v in kw.items()]
    if backend is not None:
        parts.append(f"backend={backend!r}")
    return ", ".join(parts)


def generate_profile_script(op_name: str, kernel_name: str, pos: list, kw: dict) -> str:
    cls = op_name_to_class(op_name)
    backend = None if kernel_name == "ref" else kernel_name
    call = "op._ref_forward(*data)" if kernel_name == "ref" else "op(*data)"
    return textwrap.dedent(f"""\
        import sys
        sys.path.insert(0, {str(ROOT)!r})
        import torch
        from {PACKAGE} import {cls}

        op = {cls}({_ctor_args(pos, kw, backend)})
        data = op.gen_data()
        {call}
        torch.cuda.synchronize()
    """)


def _op_class(op_name: str):
    return getattr(importlib.import_module(PACKAGE), op_name_to_class(op_name))


def show_help_no_op() -> None:
    print(__doc__)
    from ezops_b200 import list_ops

    print("Available ops:")
    for name in list_ops():
        print(f"  {name}")


def show_help_for_op(op_name: str) -> None:
    from ezops_b200 import list_backends

    try:
        cls = _op_class(op_name)
    except (ImportError, AttributeError) as exc:
        print(f"Error: unknown op {op_name!r}: {exc}")
        sys.exit(1)
    print(f"Op: {op_name} ({cls.__name__})\n\nAvailable kernels:")
    for k in ["ref"] + list_backends(op_name):
        print(f"  {k}")
    desc = getattr(cls, "_params_desc", {})
    print("\nParameters:" if desc else "\nParameters: (no description available)")
    for name, text in desc.items():
        print(f"  {name}  {text}")
    if desc:
        print(f"\nExample: -p {','.join(f'{k}=<{k}>' for k in desc)}")


def warmup(op_name: str, kernel_name: str, pos: list, kw: dict, n: int) -> None:
    import torch

    backend = None if kernel_name == "ref" else kernel_name
    op = _op_class(op_name)(*pos, **kw, **({"backend": backend} if backend else {}))
    data = op.gen_data()
    fn = op._ref_forward if kernel_name == "ref" else op.__call__
    for _ in range(n):
        fn(*data)
    torch.cuda.synchronize()


def ncu_command(ncu: str, output: Path, script: Path, launches: int, kernel_regex: str | None) -> list[str]:
    cmd = [ncu, "--set", "full", "--clock-control", "none", "-c", str(launches), "-o", str(output), "--force-overwrite"]
    if kernel_regex:
        cmd += ["-k", f"regex:{kernel_regex}"]
    return cmd + [sys.executable, str(script)]


def main():
    if "-h" in sys.argv or "--help" in sys.argv:
        rest = [a for a in sys.argv[1:] if a not in ("-h", "--help")]
        show_help_for_op(rest[0]) if rest else show_help_no_op()
        sys.exit(0)
    ap = argparse.ArgumentParser(description="Profile operator kernels with Nsight Compute")
    ap.add_argument("op_name")
    ap.add_argument("--kernels", "-k", default="ref")
    ap.add_argument("--output-dir", "-o", default=".profiles")
    ap.add_argument("--params", "-p", default="")
    ap.add_argument("--warmup", "-w", type=int, default=10)
    ap.add_argument("--launches", "-c", type=int, default=3, help="kernel launches to capture (default 3)")
    ap.add_argument("--kernel-regex", "-K", default=None, help="capture only kernels whose name matches")
    args = ap.parse_args()

    ncu = shutil.which("ncu")
    if ncu is None:
        print("Error: ncu not found on PATH.")
        sys.exit(1)
    try:
        _op_class(args.op_name)
    except (ImportError, AttributeError) as exc:
        print(f"Error: cannot import {op_name_to_class(args.op_name)} from {PACKAGE}: {exc}")
        sys.exit(1)
    if args.kernels == "all":
        from ezops_b200 import list_backends

        kernels = ["ref"] + list_backends(args.op_name)
    else:
        kernels = [k.strip() for k in args.kernels.split(",")]
    out_dir = Path(args.output_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    pos, kw = parse_params(args.params)

    for kernel_name in kernels:
        label = f"{args.op_name}/{kernel_name}"
        print(f"\nWarming up {label} ({args.warmup} iters) ...")
        try:
            warmup(args.op_name, kernel_name, pos, kw, args.warmup)
        except Exception as exc:
            print(f"Warning: warmup failed: {exc}")
        script = out_dir / f"_run_{args.op_name}_{kernel_name}.py"
        script.write_text(generate_profile_script(args.op_name, kernel_name, pos, kw))
        plain = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=300)
        if plain.returncode != 0:
            print(f"  not profiled: the plain run of {label} exited {plain.returncode}")
            for line in plain.stderr.strip().splitlines()[-5:]:
                print(f"  {line}")
            script.unlink(missing_ok=True)
            continue
        print(f"Profiling {label} ...")
        output = out_dir / f"{args.op_name}_{kernel_name}_{datetime.now().strftime('%Y%m%d_%H%M%S')}"
        result = subprocess.run(ncu_command(ncu, output, script, args.launches, args.kernel_regex), capture_output=True, text=True)
        if result.returncode != 0:
            print(f"  FAILED (exit {result.returncode})")
            for line in result.stderr.strip().splitlines()[-5:]:
                print(f"  {line}")
        else:
            rep = output.with_suffix(".ncu-rep")
            print(f"  Saved: {rep} ({rep.stat().st_size / 1024:.1f} KB)" if rep.exists() else f"  Done (see {out_dir}/)")
        script.unlink(missing_ok=True)
    print(f"\nDone. Reports in {out_dir}/")


if __name__ == "__main__":
    main()
