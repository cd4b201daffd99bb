"""Position encodings.  A mixer builds the one its spec names and asks it for per-step tables."""
from __future__ import annotations

from typing import Any, Dict, Tuple

import torch

from ..csrc import kernels as K
from .base import Runtime, StepContext
from .registry import register_position


@register_position("rope_neox")
class RotaryNeoX:
    """Rotary positions with NeoX pairing (i, i + rotary_dim/2): angle = pos * theta^(-2i/rotary_dim)
    (pkg/ops/rope_tables.go:6-20, pkg/ops/rope_heads.go:30-38).  Angles, cos and sin are computed in
    float64 once per step for all layers that share (theta, rotary_dim) and stored as float32."""

    def __init__(self, params: Dict[str, Any], rt: Runtime):
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {self.rotary_dim}")
        half = self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64),
                                  -2.0 * i / self.rotary_dim).to(rt.device)
        self.key = ("rope_neox", self.theta, self.rotary_dim)

    def tables(self, ctx: StepContext) -> Tuple[torch.Tensor, torch.Tensor]:
        got = ctx.shared.get(self.key)
        if got is None:
            half = self.rotary_dim // 2
            cos = ctx.ws.get(f"rope_cos_{self.theta}_{self.rotary_dim}", (ctx.n_tokens, half), torch.float32)
            sin = ctx.ws.get(f"rope_sin_{self.theta}_{self.rotary_dim}", (ctx.n_tokens, half), torch.float32)
            K.rope_tables(ctx.positions, self.inv_freq, cos, sin)
            got = ctx.shared[self.key] = (cos, sin)
        return got
