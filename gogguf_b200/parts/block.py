"""Block arrangements: how a mixer, a feed-forward and their norms are wired around the residual."""
from __future__ import annotations

import torch

from ..config.spec import BlockSpec
from .base import Runtime, StepContext
from .registry import register_arrangement


@register_arrangement("pre_norm")
class PreNormBlock:
    """x += mixer(norm1(x)); x += feed_forward(norm2(x)) (pkg/model/qwen3/model.go:198-288).
    The residual stream x is float32; the parts add their outputs into it."""

    def __init__(self, spec: BlockSpec, mixer, feed_forward, mixer_norm, feed_forward_norm, rt: Runtime):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.rt = rt

    def forward(self, x: torch.Tensor, ctx: StepContext, cache, writes_cache: bool) -> None:
        h = ctx.ws.get("block_normed", tuple(x.shape), self.rt.dtype)
        self.mixer_norm.forward(x, h)
        self.mixer.forward(h, x, ctx, cache, writes_cache)
        self.feed_forward_norm.forward(x, h)
        self.feed_forward.forward(h, x, ctx)
