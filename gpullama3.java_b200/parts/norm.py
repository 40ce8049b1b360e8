"""RMSNorm, the only norm of the Llama 3 decoder (inference/InferenceCore.java:47-56 of the
reference project): used before the mixer, before the feed-forward and before the output head."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import Norm, register_norm


class RMSNorm(Norm):
    graph_safe = True
    pad_safe = True

    def __init__(self, dim: int, eps: float):
        self.dim, self.eps = int(dim), float(eps)
        self.weight: torch.Tensor | None = None

    def parameters(self):
        return {"weight": ParamSpec((self.dim,), "norm")}

    def load(self, tensors, dtype, device):
        w = tensors["weight"]
        # a weight stored in 32 bits stays so; the float32 run takes everything in 32 bits
        keep = torch.float32 if (dtype == torch.float32 or w.dtype == torch.float32) else torch.bfloat16
        self.weight = w.to(device=device, dtype=keep).contiguous()

    def row_factor_form(self):
        return self.weight, self.eps, self.dim

    def forward(self, x, out_dtype, rows=None, alloc=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = alloc((n, self.dim), out_dtype) if alloc is not None else torch.empty((n, self.dim), dtype=out_dtype, device=x.device)
        ops.rmsnorm(x, self.weight, out, self.eps, rows)
        return out


register_norm("rmsnorm", RMSNorm)
