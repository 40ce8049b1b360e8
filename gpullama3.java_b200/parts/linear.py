"""A weight matrix [out, in] and the choice of kernel that multiplies activations with it.

The kernels are chosen by precision and size only (the true 32-bit run always takes the plain FMA
kernel; the bfloat16 run takes a tensor-core kernel where one accepts the sizes), never by
model."""
from __future__ import annotations

import torch

from ..kernels import fast, ops
from .base import ScaledRows


class Linear:
    def __init__(self, weight: torch.Tensor):
        assert weight.dim() == 2 and weight.is_contiguous()
        self.weight = weight
        self.out_features, self.in_features = weight.shape

    def _run(self, a, c: torch.Tensor, epilogue: int) -> None:
        if isinstance(a, ScaledRows):  # only handed to a product that said it links (links_with)
            ops.gemm_decode_linked(a.data, self.weight, c, epilogue, row_factors=(a.partials, a.eps, a.dim))
            return
        if fast.try_gemm(a, self.weight, c, epilogue):
            return
        ops.gemm_generic(a, self.weight, c, epilogue)

    def links_with(self, n_rows: int, dtype: torch.dtype) -> bool:
        """Whether this product can be one half of a split norm for ``n_rows`` rows of ``dtype``."""
        return dtype == torch.bfloat16 and ops.gemm_decode_links(n_rows, self.weight)

    def store(self, a: torch.Tensor, out_dtype: torch.dtype, alloc=None) -> torch.Tensor:
        """a @ W.T as a new [T, out] tensor (from ``alloc(shape, dtype)`` when given, a step's ``ctx.empty``)."""
        shape = (a.shape[0], self.out_features)
        c = alloc(shape, out_dtype) if alloc is not None else torch.empty(shape, dtype=out_dtype, device=a.device)
        self._run(a, c, ops.EPILOGUE_STORE)
        return c

    def into(self, a: torch.Tensor, c: torch.Tensor) -> None:
        """c = a @ W.T into a tensor the caller brings."""
        self._run(a, c, ops.EPILOGUE_STORE)

    def add_to(self, a: torch.Tensor, residual: torch.Tensor, then_norm=None) -> ScaledRows | None:
        """residual += a @ W.T, the sum kept in float32.  With ``then_norm`` (a norm that has a row-factor form)
        and a product that links, the same kernel also leaves that norm of the new residual as ScaledRows."""
        form = then_norm.row_factor_form() if then_norm is not None else None
        if (form is not None and a.dtype == torch.bfloat16 and self.links_with(a.shape[0], a.dtype)
                and form[2] == self.out_features and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0):
            weight, eps, dim = form
            n = a.shape[0]
            act = torch.empty((n, dim), dtype=torch.bfloat16, device=a.device)
            partials = torch.empty((n, ops.gemm_decode_partials(n, self.out_features)), dtype=torch.float32, device=a.device)
            ops.gemm_decode_linked(a, self.weight, residual, ops.EPILOGUE_RESIDUAL_ADD, emit=(weight, act, partials))
            return ScaledRows(act, partials, eps, dim)
        self._run(a, residual, ops.EPILOGUE_RESIDUAL_ADD)
        return None

    def gated_silu(self, a: torch.Tensor, out_dtype: torch.dtype, alloc=None) -> torch.Tensor:
        """W holds gate and up rows interleaved; returns silu(gate) * up as [T, out/2]."""
        shape = (a.shape[0], self.out_features // 2)
        c = alloc(shape, out_dtype) if alloc is not None else torch.empty(shape, dtype=out_dtype, device=a.device)
        self._run(a, c, ops.EPILOGUE_GATED_SILU)
        return c
