"""How a mixer and a feed-forward are arranged into one block."""

from __future__ import annotations

import torch

from oxr_inference_b200.parts.base import ARRANGEMENTS, DeferredLinear, FeedForward, LayerCache, Mixer, Norm, StepContext


@ARRANGEMENTS.register("pre_norm")
class PreNormBlock:
    """``x += mixer(norm1(x)); x += feed_forward(norm2(x))``, carried as (last output not yet added, residual):
    each norm first adds the pending output into the fp32 residual stream (oxr_runtime/language.py:184-187,
    253-257,266-269). Returns the feed-forward's output and the residual; whoever comes next adds them.

    Two optional hand-overs take the norm kernels out of a decode step; each happens only when both sides say that they can.
    A norm that ``accepts_deferred`` gets the part before it with its last projection still to do (:class:`DeferredLinear`;
    with ``defer_output`` the block's own output is left like that for the next block's norm, which the decoder asks for only
    when the next block ``accepts_deferred_input``), so that the product can add itself into the residual stream. And when
    the part behind such a norm ``accepts_lazy_input``, the norm may hand it a not yet normalised ``h`` that its first
    projection normalises itself."""

    supports_deferred = True

    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward, feed_forward_norm: Norm):
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm

    def parts(self) -> dict[str, object]:
        return {"mixer": self.mixer, "mixer_norm": self.mixer_norm, "feed_forward": self.feed_forward,
                "feed_forward_norm": self.feed_forward_norm}

    @property
    def accepts_deferred_input(self) -> bool:
        return bool(self.mixer_norm.accepts_deferred)

    @staticmethod
    def _norm(norm: Norm, x, residual, behind) -> tuple:
        if norm.accepts_deferred:
            return norm.forward(x, residual, lazy=bool(getattr(behind, "accepts_lazy_input", False)))
        if isinstance(x, DeferredLinear):
            x = x.materialize()
        return norm.forward(x, residual)

    def forward(self, x, residual: torch.Tensor | None, ctx: StepContext, cache: LayerCache, defer_output: bool = False):
        h, residual = self._norm(self.mixer_norm, x, residual, self.mixer)
        if self.feed_forward_norm.accepts_deferred:
            a = self.mixer.forward_deferred(h, ctx, cache)
        else:
            a = self.mixer.forward(h, ctx, cache)
        h, residual = self._norm(self.feed_forward_norm, a, residual, self.feed_forward)
        return (self.feed_forward.forward_deferred(h) if defer_output else self.feed_forward.forward(h)), residual
