"""Block arrangements: how a mixer, a feed-forward and their norms are wired around the residual."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import BlockSpec
from .base import RowStats, Runtime, StepContext
from .registry import register_arrangement


@register_arrangement("pre_norm")
class PreNormBlock:
    """x += mixer(norm1(x)); x += feed_forward(norm2(x)) (pkg/model/qwen3/model.go:198-288).
    The residual stream x is float32; the parts add their outputs into it."""

    # role -> family: what a block of this arrangement is made of (the builder builds exactly these)
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}
    keeps_row_stats = True      # clears RowStats.fresh itself before each write to the residual

    def __init__(self, spec: BlockSpec, parts: Dict[str, object], rt: Runtime):
        self.parts = dict(parts)
        mixer, feed_forward = parts["mixer"], parts["feed_forward"]
        mixer_norm, feed_forward_norm = parts["mixer_norm"], parts["feed_forward_norm"]
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.rt = rt
        # A part may take its pre-norm into its first projection (`absorb_norm(norm) -> bool`); it then
        # gets the residual's RowStats as `h` instead of normalised rows, and the norm kernel does not run.
        self.mixer_folded = _offer_norm(mixer, mixer_norm, rt)
        self.feed_forward_folded = _offer_norm(feed_forward, feed_forward_norm, rt)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache, writes_cache: bool) -> None:
        stats = ctx.shared.get("row_stats")
        if stats is None and (self.mixer_folded or self.feed_forward_folded):
            T, H = x.shape
            stats = ctx.shared["row_stats"] = RowStats(
                ctx.ws.get("residual_bf16", (T, H), torch.bfloat16),
                ctx.ws.get("residual_ssq", (T, (H + 127) // 128), torch.float32))
        h = self._input(self.mixer_folded, self.mixer_norm, x, ctx, stats)
        self.mixer.forward(h, x, ctx, cache, writes_cache)
        h = self._input(self.feed_forward_folded, self.feed_forward_norm, x, ctx, stats)
        self.feed_forward.forward(h, x, ctx)

    def _input(self, folded: bool, norm, x: torch.Tensor, ctx: StepContext, stats):
        if folded:
            h = stats.ensure(x)
        else:
            h = ctx.ws.get("block_normed", tuple(x.shape), self.rt.dtype)
            norm.forward(x, h)
        if stats is not None:
            stats.fresh = False        # the part is about to change the residual rows
        return h


def _offer_norm(part, norm, rt: Runtime) -> bool:
    absorb = getattr(part, "absorb_norm", None)
    if absorb is None or not (rt.fast and rt.fold_norms and rt.dtype == torch.bfloat16):
        return False
    if not getattr(norm, "foldable", False):
        return False
    return bool(absorb(norm))
