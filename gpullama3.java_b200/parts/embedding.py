"""Token embedding and the output head.

The embedding copies a table row into the residual stream (inference/InferenceCore.java:69 of the
reference project); the head multiplies the normalised rows whose logits are wanted with the
classifier matrix, which is the embedding table itself when the model ties them
(model/loader/ModelLoader.java:253)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import Part
from .linear import Linear


class TokenEmbedding(Part):
    graph_safe = True
    pad_safe = True

    def __init__(self, vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.table: torch.Tensor | None = None

    def parameters(self):
        return {"table": ParamSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors, dtype, device):
        t = tensors["table"].to(device)
        self.table = t.to(torch.float32 if dtype == torch.float32 else t.dtype).contiguous()

    def forward(self, tokens: torch.Tensor, alloc=None) -> torch.Tensor:
        shape = (tokens.numel(), self.hidden_size)
        out = alloc(shape, torch.float32) if alloc is not None else torch.empty(shape, dtype=torch.float32, device=tokens.device)
        ops.embed_gather(self.table, tokens, out)
        return out


class OutputHead(Part):
    graph_safe = True
    pad_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: TokenEmbedding | None = None):
        self.vocab_size, self.hidden_size, self.tied_to = vocab_size, hidden_size, tied_to
        self.linear: Linear | None = None

    def parameters(self):
        return {} if self.tied_to is not None else {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors, dtype, device):
        if self.tied_to is not None:
            self.linear = Linear(self.tied_to.table)  # the same device memory as the embedding
        else:
            w = tensors["weight"].to(device)
            self.linear = Linear(w.to(torch.float32 if dtype == torch.float32 else w.dtype).contiguous())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: normalised rows [R, hidden] -> float32 logits [R, vocab]."""
        return self.linear.store(x, torch.float32)
