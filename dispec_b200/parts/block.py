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

    # RMSNorm applied inside the first product of the mixer / feed-forward (few rows only).
    # Off: measured slower than a norm kernel of its own followed by the plain product.
    fuse_norm_into_linear = False

    def _takes_residual(self) -> bool:
        return (getattr(self.mixer, "fuses_norm_and_residual", False)
                and getattr(self.feed_forward, "fuses_norm_and_residual", False))

    def _norm_fusable(self, x) -> bool:
        from dispec_b200.ops import gemm
        return (self.fuse_norm_into_linear and gemm.fused_prologue_supported(x, x)
                and hasattr(self.mixer_norm, "as_linear_prologue")
                and hasattr(self.ffn_norm, "as_linear_prologue"))

    def forward(self, ctx, x, pending, cache, state):
        if pending is None and self._takes_residual():
            # the sums into the residual stream happen in the epilogue of the last product of the
            # mixer and of the feed-forward (32-bit sum, rounded once)
            if self._norm_fusable(x):
                x = self.mixer.forward(ctx, x, cache, state, pre_norm=self.mixer_norm, residual=x)
                x = self.feed_forward.forward(ctx, x, pre_norm=self.ffn_norm, residual=x)
            else:
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
