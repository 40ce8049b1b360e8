"""The dense gated feed-forward of the Llama 3 decoder (SwiGLU):
down( silu(gate(x)) * up(x) ), inference/InferenceCore.java:154-172 of the reference project.
Gate and up rows are interleaved into one weight at load so that one matrix product's epilogue
sees a gate value and its up value side by side (the reference fuses the same pair in one kernel,
tornadovm/TransformerComputeKernelsLayered.java:808-826)."""
from __future__ import annotations

import torch

from ..weights.loader import ParamSpec
from .base import FeedForward, StepContext, register_feed_forward
from .linear import Linear


class SwiGLUFeedForward(FeedForward):
    graph_safe = True
    pad_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_up: Linear | None = None
        self.down: Linear | None = None

    def parameters(self):
        return {"gate": ParamSpec((self.intermediate_size, self.hidden_size)),
                "up": ParamSpec((self.intermediate_size, self.hidden_size)),
                "down": ParamSpec((self.hidden_size, self.intermediate_size))}

    def load(self, tensors, dtype, device):
        gate, up, down = (tensors[n].to(device) for n in ("gate", "up", "down"))
        common = torch.float32 if (dtype == torch.float32 or torch.float32 in (gate.dtype, up.dtype)) else gate.dtype
        fused = torch.stack([gate.to(common), up.to(common)], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        self.gate_up = Linear(fused.contiguous())
        self.down = Linear(down.to(torch.float32 if dtype == torch.float32 else down.dtype).contiguous())

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        return ctx.all_decode and self.gate_up.links_with(ctx.n_tokens, ctx.dtype)

    def forward(self, x, ctx: StepContext, residual, then_norm=None):
        h = self.gate_up.gated_silu(x, ctx.dtype, ctx.empty)  # [T, intermediate]
        return self.down.add_to(h, residual, then_norm)


register_feed_forward("swiglu", SwiGLUFeedForward)
