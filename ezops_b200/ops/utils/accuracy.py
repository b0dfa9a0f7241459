"""Untimed acceptance checks run before a kernel is timed
(ezops/ops/utils/accuracy.py:19-78): signal-to-noise of one call against the
reference, two-call byte-for-byte determinism, and inputs left untouched."""

from __future__ import annotations

import math
from collections.abc import Callable, Iterable

import torch

SQNR_THRESHOLD_DB = 28.0


def sqnr_db(ref: torch.Tensor, out: torch.Tensor) -> float:
    """10*log10(|ref|^2 / |ref-out|^2); ``inf`` for an exact match."""
    r = ref.detach().float()
    err = (r - out.detach().float()).square().sum().item()
    if err == 0.0:
        return math.inf
    return 10.0 * math.log10(r.square().sum().item() / err)


def _raw(t: torch.Tensor) -> torch.Tensor:
    return t.detach().contiguous().reshape(-1).view(torch.uint8)


def bitwise_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Equality of the stored bytes (so -0.0 != +0.0 and NaN payloads count)."""
    return a.shape == b.shape and a.dtype == b.dtype and bool(torch.equal(_raw(a), _raw(b)))


def _tup(x) -> tuple:
    return (x,) if isinstance(x, torch.Tensor) else tuple(x)


def check_determinism(fn: Callable, inputs: Iterable[torch.Tensor], outputs) -> bool:
    ins, outs = _tup(inputs), _tup(outputs)
    fn(*ins, *outs)
    snapshot = [o.clone() for o in outs]
    fn(*ins, *outs)
    return all(bitwise_equal(o, s) for o, s in zip(outs, snapshot, strict=True))


def check_input_readonly(fn: Callable, inputs: Iterable[torch.Tensor], outputs) -> bool:
    ins, outs = _tup(inputs), _tup(outputs)
    saved = [i.clone() for i in ins]
    fn(*ins, *outs)
    return all(bitwise_equal(i, s) for i, s in zip(ins, saved, strict=True))


def bf16_ulp_mismatch(actual: torch.Tensor, expected: torch.Tensor) -> dict:
    """How far two bf16 tensors are apart in units of the last place: the
    histogram ``{0: n_equal, 1: n_one_ulp, ">1": n_more}`` over all elements."""
    a = actual.detach().contiguous().view(torch.int16).to(torch.int32)
    e = expected.detach().contiguous().view(torch.int16).to(torch.int32)
    # map sign-magnitude bf16 bit patterns to a monotone integer line
    a = torch.where(a < 0, -(a & 0x7FFF), a)
    e = torch.where(e < 0, -(e & 0x7FFF), e)
    d = (a - e).abs()
    return {0: int((d == 0).sum()), 1: int((d == 1).sum()), ">1": int((d > 1).sum())}
