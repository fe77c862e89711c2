"""RMSNorm fused with the residual add: y = x * rsqrt(mean(x^2) + eps) * w with the
weight multiplying directly (no 1 + w), sums in float32
(reference: src/cuda/kernels/elementwise.cu:29-64)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..ops import kernels
from .base import Norm, register
from .spec import TensorSpec


@dataclass(frozen=True)
class RMSNormParams:
    size: int
    eps: float


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    def tensors(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.params.size,))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def add_norm(self, residual, delta, out, rows_idx=None, rows=None) -> None:
        kernels.add_rmsnorm(residual, delta, self.weight, out, self.params.eps, rows_idx, rows)

    def rms_params(self):
        return self.weight, self.params.eps
