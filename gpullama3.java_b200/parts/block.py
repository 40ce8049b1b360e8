"""The pre-norm residual block: x += mixer(norm(x)); x += feed_forward(norm(x)), the order of
inference/InferenceCore.java:72-173 of the reference project.  The residual stream is float32."""
from __future__ import annotations

from .base import Block, StepContext, register_block


class PreNormBlock(Block):
    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.children().values())

    def forward(self, residual, ctx: StepContext, cache, writes_cache=True):
        self.mixer.forward(self.mixer_norm.forward(residual, ctx.dtype), ctx, cache, residual, writes_cache)
        self.feed_forward.forward(self.feed_forward_norm.forward(residual, ctx.dtype), ctx, residual)


register_block("pre_norm", PreNormBlock)
