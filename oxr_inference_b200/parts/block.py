"""How a mixer and a feed-forward are arranged into one block."""

from __future__ import annotations

import torch

from oxr_inference_b200.parts.base import ARRANGEMENTS, FeedForward, LayerCache, Mixer, Norm, StepContext


@ARRANGEMENTS.register("pre_norm")
class PreNormBlock:
    """``x += mixer(norm1(x)); x += feed_forward(norm2(x))``, carried as (last output not yet added, residual):
    each norm first adds the pending output into the fp32 residual stream (oxr_runtime/language.py:184-187,
    253-257,266-269). Returns the feed-forward's output and the residual; whoever comes next adds them."""

    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward, feed_forward_norm: Norm):
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm

    def parts(self) -> dict[str, object]:
        return {"mixer": self.mixer, "mixer_norm": self.mixer_norm, "feed_forward": self.feed_forward,
                "feed_forward_norm": self.feed_forward_norm}

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext, cache: LayerCache):
        h, residual = self.mixer_norm.forward(x, residual)
        a = self.mixer.forward(h, ctx, cache)
        h, residual = self.feed_forward_norm.forward(a, residual)
        return self.feed_forward.forward(h), residual
