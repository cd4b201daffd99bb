"""Dense SwiGLU feed-forward: down( silu(gate h) * (up h) ), no bias
(pkg/model/qwen3/model.go:273-286, pkg/ops/inplace.go:14-19)."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU:
    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        h, i = spec["hidden_size"], spec["intermediate_size"]
        return {
            "gate_proj.weight": TensorDecl(shape=(i, h)),
            "up_proj.weight": TensorDecl(shape=(i, h)),
            "down_proj.weight": TensorDecl(shape=(h, i)),
        }

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        g, u = rt.matrix(weights["gate_proj.weight"]), rt.matrix(weights["up_proj.weight"])
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.rt = rt
        self.fused = None
        if (rt.fast and rt.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and self.inter % 64 == 0
                and self.inter >= 128 and self.hidden % 8 == 0):
            # gate and up rows interleaved in blocks of 64: the product's epilogue applies silu(gate) * up
            # and writes the activation directly, so the [T, 2 I] intermediate never exists
            from ..csrc import tcgen05_gemm
            self.fused = Linear(tcgen05_gemm.interleave_gate_up(g, u), rt, swiglu=True)
        if self.fused is None:
            # gate rows first, then up rows: one product for both, then the activation kernel
            self.gate_up = Linear(torch.cat([g, u], dim=0), rt)
        self.down = Linear(weights["down_proj.weight"], rt)

    def absorb_norm(self, norm) -> bool:
        """Take the block's pre-norm into the gate/up projection; `forward` then gets RowStats as `h`."""
        first = self.fused if self.fused is not None else self.gate_up
        if not first.can_fold or norm.size != self.hidden:
            return False
        first.fold_input_norm(norm.weight, norm.eps)
        return True

    def forward(self, h, residual: torch.Tensor, ctx: StepContext) -> None:
        T = ctx.n_tokens
        act = ctx.ws.get("ffn_act", (T, self.inter), self.rt.dtype)
        if self.fused is not None:
            self.fused(h, act, ws=ctx.ws)
        else:
            gu = ctx.ws.get("ffn_gate_up", (T, 2 * self.inter), self.rt.dtype)
            self.gate_up(h, gu, ws=ctx.ws)
            K.swiglu(gu, act, T, self.inter)
        self.down(act, residual, accumulate=True, ws=ctx.ws, emit=ctx.shared.get("row_stats"))
