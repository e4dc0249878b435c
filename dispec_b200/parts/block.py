"""Arrangement of a layer: pre-norm residual block.

    x += pending;  h = norm1(x);  a = mixer(h);  x += a;  h = norm2(x);  pending = ffn(h)

(puneethgv/DiSpec dispec/engine/model_runner.py:214-219).  The sum into the residual stream
is fused into the norm that follows it and computed in 32-bit; the block hands the last
feed-forward output on as ``pending`` so that the next block's first norm (or the final norm)
adds it."""
from __future__ import annotations

from dispec_b200.ops.gemm import NormedRows
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

    def _defers_norms(self) -> bool:
        return (self._takes_residual() and hasattr(self.mixer_norm, "deferred")
                and hasattr(self.ffn_norm, "after_product")
                and getattr(self.mixer, "takes_deferred_norm", False)
                and getattr(self.feed_forward, "takes_deferred_norm", False))

    def first_norm_after_product(self):
        """(weight, eps) of this block's first norm if the block takes that norm as ``pending``
        (a ``NormedRows`` of its ``x``) from whoever wrote ``x``; else None."""
        if self._defers_norms() and hasattr(self.mixer_norm, "after_product"):
            return self.mixer_norm.after_product()
        return None

    def forward(self, ctx, x, pending, cache, state, then_norm=None):
        """``then_norm``: (weight, eps) of the norm that reads this block's result first (the next
        block's, offered by its ``first_norm_after_product``); a block that can hands back that
        norm, still to be applied, as ``pending``."""
        if self._defers_norms() and (pending is None or isinstance(pending, NormedRows)):
            # each norm is handed to the product after it, which takes it apart where it can: the
            # product before stores the rows times the gain beside its result, the product after
            # scales its own result rows (see ops.gemm.NormedRows); else the norm kernel runs there
            h = pending if pending is not None else self.mixer_norm.deferred(x)
            x, h = self.mixer.forward(ctx, h, cache, state, residual=x,
                                      then_norm=self.ffn_norm.after_product())
            if then_norm is None:
                return self.feed_forward.forward(ctx, h, residual=x), None
            return self.feed_forward.forward(ctx, h, residual=x, then_norm=then_norm)
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
