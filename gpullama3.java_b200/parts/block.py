"""The pre-norm residual block: x += mixer(norm(x)); x += feed_forward(norm(x)), the order of
inference/InferenceCore.java:72-173 of the reference project.  The residual stream is float32."""
from __future__ import annotations

from .base import Block, StepContext, all_parts, register_block


class PreNormBlock(Block):
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm):
        super().__init__(mixer=mixer, feed_forward=feed_forward, mixer_norm=mixer_norm,
                         feed_forward_norm=feed_forward_norm)

    @property
    def graph_safe(self):
        # the block itself launches nothing; its decode step is as replayable as its parts' launches are
        return all(p.graph_safe for p in all_parts(self).values())

    @property
    def pad_safe(self):
        return all(p.pad_safe for p in all_parts(self).values())

    def first_norm(self):
        return self.mixer_norm

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        return self.mixer.takes_scaled_rows(ctx) and self.mixer_norm.row_factor_form() is not None

    def forward(self, residual, ctx: StepContext, cache, writes_cache=True, x_in=None, then_norm=None):
        """In a decode step the two norms need not be kernels of their own: the product that completes the
        residual stream before a norm (the mixer's, or the previous block's, last product) leaves the norm's
        rows one factor short, and the product after it applies the factor (ScaledRows).  Parts that do not
        offer this are called the plain way."""
        x = x_in if x_in is not None else self.mixer_norm.forward(residual, ctx.dtype, alloc=ctx.empty)
        h = None
        if self.mixer.takes_scaled_rows(ctx):
            ffn_links = self.feed_forward.takes_scaled_rows(ctx)
            h = self.mixer.forward(x, ctx, cache, residual, writes_cache,
                                   then_norm=self.feed_forward_norm if ffn_links else None)
        else:
            self.mixer.forward(x, ctx, cache, residual, writes_cache)
        if h is None:
            h = self.feed_forward_norm.forward(residual, ctx.dtype, alloc=ctx.empty)
        if self.feed_forward.takes_scaled_rows(ctx):
            return self.feed_forward.forward(h, ctx, residual, then_norm=then_norm)
        self.feed_forward.forward(h, ctx, residual)
        return None


register_block("pre_norm", PreNormBlock)
