"""A weight matrix [out, in] and the choice of kernel that multiplies activations with it.

The kernels are chosen by precision and size only (the true 32-bit run always takes the plain FMA
kernel; the bfloat16 run takes a tensor-core kernel where one accepts the sizes), never by
model."""
from __future__ import annotations

import torch

from ..kernels import ops


class Linear:
    def __init__(self, weight: torch.Tensor):
        assert weight.dim() == 2 and weight.is_contiguous()
        self.weight = weight
        self.out_features, self.in_features = weight.shape

    def _run(self, a: torch.Tensor, c: torch.Tensor, epilogue: int) -> None:
        from ..kernels import fast

        if fast.try_gemm(a, self.weight, c, epilogue):
            return
        ops.gemm_generic(a, self.weight, c, epilogue)

    def store(self, a: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """a @ W.T as a new [T, out] tensor."""
        c = torch.empty((a.shape[0], self.out_features), dtype=out_dtype, device=a.device)
        self._run(a, c, ops.EPILOGUE_STORE)
        return c

    def add_to(self, a: torch.Tensor, residual: torch.Tensor) -> None:
        """residual += a @ W.T, the sum kept in float32."""
        self._run(a, residual, ops.EPILOGUE_RESIDUAL_ADD)

    def gated_silu(self, a: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """W holds gate and up rows interleaved; returns silu(gate) * up as [T, out/2]."""
        c = torch.empty((a.shape[0], self.out_features // 2), dtype=out_dtype, device=a.device)
        self._run(a, c, ops.EPILOGUE_GATED_SILU)
        return c
