"""Shared test helpers: golden-fixture loading and comparison metrics."""

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_golden(name: str) -> dict:
    """Load ``tests/golden/<name>.npz``; uint16 arrays are bf16 bit patterns."""
    out = {}
    with np.load(GOLDEN / f"{name}.npz") as z:
        for key in z.files:
            a = z[key]
            if a.dtype == np.uint16:
                out[key] = torch.from_numpy(a.copy()).view(torch.bfloat16)
            elif a.ndim == 0:
                out[key] = a.item()
            else:
                out[key] = torch.from_numpy(a.copy())
    return out


def rel_fro(a: torch.Tensor, e: torch.Tensor) -> float:
    a, e = a.detach().double().cpu(), e.detach().double().cpu()
    return ((a - e).norm() / max(e.norm().item(), 1e-30)).item()


def max_abs(a: torch.Tensor, e: torch.Tensor) -> float:
    return (a.detach().double().cpu() - e.detach().double().cpu()).abs().max().item()


def ulp_hist(a: torch.Tensor, e: torch.Tensor) -> dict:
    from ezops_b200.ops.utils.accuracy import bf16_ulp_mismatch

    return bf16_ulp_mismatch(a.detach().cpu(), e.detach().cpu())


def frac_within_one_ulp(a: torch.Tensor, e: torch.Tensor) -> float:
    h = ulp_hist(a, e)
    n = h[0] + h[1] + h[">1"]
    return (h[0] + h[1]) / max(n, 1)
