"""Arrangement of a layer: pre-norm residual block.

    x += pending;  h = norm1(x);  a = mixer(h);  x += a;  h = norm2(x);  pending = ffn(h)

(puneethgv/DiSpec dispec/engine/model_runner.py:214-219).  The sum into the residual stream
is fused into the norm that follows it and computed in 32-bit; the block hands the last
feed-forward output on as ``pending`` so that the next block's first norm (or the final norm)
adds it."""
from __future__ import annotations

from dispec_b200.parts.base import Block
from dispec_b200.registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    def __init__(self, mixer_norm, mixer, ffn_norm, feed_forward):
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ffn_norm = ffn_norm
        self.feed_forward = feed_forward

    def _takes_residual(self) -> bool:
        return (getattr(self.mixer, "adds_residual", False)
                and getattr(self.feed_forward, "adds_residual", False))

    def forward(self, ctx, x, pending, cache, state):
        if pending is None and self._takes_residual():
            # the sums into the residual stream happen in the epilogue of the last product of the
            # mixer and of the feed-forward (32-bit sum, rounded once)
            h = self.mixer_norm.forward(ctx, x)
            x = self.mixer.forward(ctx, h, cache, state, residual=x)
            h = self.ffn_norm.forward(ctx, x)
            x = self.feed_forward.forward(ctx, h, residual=x)
            return x, None
        if pending is None:
            h = self.mixer_norm.forward(ctx, x)
        else:
            h = self.mixer_norm.forward_add(ctx, x, pending)
        a = self.mixer.forward(ctx, h, cache, state)
        h = self.ffn_norm.forward_add(ctx, x, a)
        return x, self.feed_forward.forward(ctx, h)
