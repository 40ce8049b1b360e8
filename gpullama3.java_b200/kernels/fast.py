"""Choice of the tensor-core kernels of the bfloat16 run.

``try_gemm`` and ``try_attention`` run the specialised sm_100a kernel that fits the operands and
return True, or return False when no specialised kernel takes these storage types or sizes (the
caller then runs the plain kernel, which takes every size).  The true 32-bit run never comes
here with anything but float32 operands and therefore always takes the plain kernels."""
from __future__ import annotations

import torch


def try_gemm(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int) -> bool:
    return False


def try_attention(qkv, out, ctx, page_table, cache, mixer) -> bool:
    return False
