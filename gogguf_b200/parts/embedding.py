"""Token embedding and the output head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..csrc import kernels as K
from ..weights.loader import TensorDecl
from .base import Linear, Runtime, StepContext
from .registry import register_embedding, register_head


@register_embedding("embedding")
class TokenEmbedding:
    """x = E[token]: a row gather into the float32 residual stream, no scaling
    (pkg/model/qwen3/model.go:169-196)."""

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl(shape=(spec["vocab_size"], spec["hidden_size"]))}

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.vocab, self.hidden = int(spec["vocab_size"]), int(spec["hidden_size"])
        self.weight = rt.matrix(weights["weight"])

    def forward(self, tokens: torch.Tensor, out: torch.Tensor) -> None:
        K.embed_gather(self.weight, tokens, out)


@register_head("linear_head")
class LinearHead:
    """logits = W h in float32; W is the embedding matrix when the spec says `tied_to`
    (pkg/model/qwen3/model.go:578-610, pkg/model/qwen3/tensors.go:36-48)."""

    @classmethod
    def tensors(cls, spec: PartSpec) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl(shape=(spec["vocab_size"], spec["hidden_size"]),
                                     optional=spec.get("tied_to") is not None)}

    def __init__(self, spec: PartSpec, weights: Dict[str, torch.Tensor], rt: Runtime,
                 tied: Optional[torch.Tensor] = None):
        self.vocab = int(spec["vocab_size"])
        if spec.get("tied_to") is not None:
            if tied is None:
                raise ValueError("head is tied but no embedding matrix was given")
            self.proj = Linear(tied, rt)
        else:
            self.proj = Linear(weights["weight"], rt)

    def forward(self, h: torch.Tensor, logits: torch.Tensor, ctx: StepContext, m: Optional[int] = None) -> None:
        self.proj(h, logits, m=m, ws=ctx.ws)
