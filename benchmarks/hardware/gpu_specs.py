"""Spec-sheet peaks of the GPUs this library targets, and profile files.

Same role and API as the reference's table (benchmarks/hardware/gpu_specs.py:17-194:
``PROFILES``, ``detect_profile``, ``get_specs``), which has no Blackwell
data-centre entry.  This library is sm_100a only, so the table holds the B200
alone.  Tensor-core figures are dense (no 2:4 sparsity), multiply and add
counted separately; HBM is the 8 TB/s spec-sheet figure the roofline fractions
of this project are quoted against.

A *profile* is a YAML file under ``assets/`` holding, per resource, the
spec-sheet ``theoretical`` value and a measured ``calibration`` factor
(written by ``benchmarks/roofline_profile.py``); ``load_profile`` returns it
with ``effective = theoretical * calibration`` filled in, which is what the
speed-of-light score divides by (benchmarks/bench_qwen3_dense_decode.py:71-95).
"""

from __future__ import annotations

from pathlib import Path

ASSETS = Path(__file__).resolve().parent.parent.parent / "assets"

PROFILES = {
    "b200": {
        "names": ["NVIDIA B200"],
        "compute_cap": "10.0",
        "hbm_bw_gb": 8000.0,
        "tensor_core_tflops": {"bf16": 2250.0, "fp16": 2250.0, "tf32": 1125.0, "fp8": 4500.0},
    },
}


def detect_profile(gpu_name: str) -> str | None:
    """Profile key for a device name as torch / nvidia-smi report it (exact,
    then either string a prefix of the other: "NVIDIA B200 180GB" still matches)."""
    names = {n: key for key, spec in PROFILES.items() for n in spec["names"]}
    if gpu_name in names:
        return names[gpu_name]
    for n, key in names.items():
        if gpu_name.startswith(n) or n.startswith(gpu_name):
            return key
    return None


def get_specs(profile: str) -> dict | None:
    return PROFILES.get(profile)


def load_profile(profile: str, assets_dir: Path | None = None) -> dict | None:
    """Read ``assets/<profile>.yaml`` and add ``effective`` to every resource that
    has a ``theoretical`` value (calibration defaults to 1)."""
    import yaml

    path = (assets_dir or ASSETS) / f"{profile}.yaml"
    if not path.exists():
        return None
    data = yaml.safe_load(path.read_text())

    def fill(node):
        if isinstance(node, dict):
            if "theoretical" in node:
                node["theoretical"] = float(node["theoretical"])
                node["calibration"] = float(node.get("calibration", 1.0))
                node["effective"] = node["theoretical"] * node["calibration"]
            for v in node.values():
                fill(v)

    fill(data)
    return data
