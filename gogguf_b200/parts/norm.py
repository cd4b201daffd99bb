"""RMSNorm: out = x * (1/sqrt(mean(x^2) + eps)) * weight (pkg/ops/rmsnorm.go:10-25)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Runtime
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm:
    # out = x / rms(x) * weight: a projection after it can take `weight` into its columns and apply
    # 1 / rms(x) to its own output rows (parts.base.RowStats)
    foldable = True

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl(shape=(spec["size"],), init="ones_normal")}

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = rt.vector(weights["weight"])

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        """x: float32 rows of the residual stream; out: compute dtype; rows: optional row gather."""
        K.rmsnorm(x, self.weight, self.eps, out, rows)
