"""Operator spec base class (ezops/ops/base_op.py:8-33).

An Op bundles the workload (constructor shape parameters + ``gen_data``), the
torch reference (``_ref_forward``, also what ``backend="ref"`` runs), the
tolerance (``check``) and a roofline estimate (``get_roofline``).
"""

from abc import ABC, abstractmethod

import torch

from .utils.roofline import RooflineResult, measure_roofline


class Op(ABC):
    _backend: str
    _atol: float = 1e-6
    _rtol: float = 1e-5
    _params_desc: dict[str, str] = {}

    @abstractmethod
    def forward(self, *args, **kwargs): ...

    @abstractmethod
    def _ref_forward(self, *args, **kwargs): ...

    @abstractmethod
    def gen_data(self): ...

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def get_roofline(self) -> RooflineResult:
        data = self.gen_data()
        if not isinstance(data, tuple):
            data = (data,)
        return measure_roofline(self._ref_forward, data, {})

    def check(self, actual, expected) -> bool:
        return torch.allclose(actual, expected, atol=self._atol, rtol=self._rtol)


def rel_frobenius(actual: torch.Tensor, expected: torch.Tensor) -> float:
    """``||a-e|| / max(||e||, 1)``: the layer ops' acceptance metric
    (ezops/ops/qwen3_dense_decode.py:64-69)."""
    diff = (actual.float() - expected.float()).norm().item()
    return diff / max(expected.float().norm().item(), 1.0)
