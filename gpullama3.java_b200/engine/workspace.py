"""Device memory for the intermediate tensors of one pass.

The reference keeps its activation buffers in the per-sequence state (``x, xb, xb2, hb, hb2, q, k, v,
att``: inference/state/State.java:28-37 of the reference project), sized once for one token.  A pass
here holds any number of tokens, so its buffers are taken from one block of device memory that is kept
between passes: nothing is asked of the allocator while a prompt runs.  There is no score buffer
(heads x context) among them; attention never materialises scores.

Use is a stack.  ``take`` hands out the next aligned piece; ``mark`` / ``release`` give back everything
taken since the mark, which the model does after every block, so a pass needs the memory of its
largest block, not of all blocks together.  Kernels run in stream order, so a piece may be handed out
again as soon as the host has released it.  When a pass needs more than the block holds, the extra
tensors come from the allocator for that pass and the block is enlarged before the next one."""
from __future__ import annotations

import math

import torch

_ALIGN = 256


class Workspace:
    def __init__(self, device, capacity: int = 0):
        self.device = torch.device(device)
        self.capacity = 0
        self._buf: torch.Tensor | None = None
        self._top = 0
        self._typed: dict = {}    # per dtype: the aligned block seen as that type, and the type's size in bytes
        self._wanted = 0          # the most a pass would have held had everything fitted
        self.overflowed = 0       # tensors that came from the allocator instead (tests and diagnostics)
        if capacity:
            self._allocate(capacity)

    def _allocate(self, nbytes: int) -> None:
        self._buf = None   # let the old block go first
        self._typed = {}
        self._buf = torch.empty(nbytes + _ALIGN, dtype=torch.uint8, device=self.device)
        self._base = (-self._buf.data_ptr()) % _ALIGN   # the first aligned byte of the block
        self.capacity = nbytes

    def reset(self) -> None:
        """A new pass begins: everything is free again; grow if the last pass did not fit."""
        if self._wanted > self.capacity:
            self._allocate(int(self._wanted * 1.25) + _ALIGN)
        self._top = 0
        self._wanted = 0

    def mark(self) -> int:
        return self._top

    def release(self, mark: int) -> None:
        if not (0 <= mark <= self._top):
            raise ValueError("workspace released to a mark that was not taken")
        self._top = mark

    def take(self, shape, dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(int(s) for s in shape)
        seen = self._typed.get(dtype)
        if seen is None:   # (pieces start on 256-byte boundaries, so every element type divides their offsets)
            size = torch.empty((), dtype=dtype).element_size()
            block = self._buf[self._base:self._base + self.capacity // size * size].view(dtype) if self._buf is not None else None
            seen = self._typed[dtype] = (block, size)
        block, size = seen
        numel = math.prod(shape)
        start = (self._top + _ALIGN - 1) // _ALIGN * _ALIGN
        end = start + numel * size
        self._top = end
        if end > self._wanted:
            self._wanted = end
        if end > self.capacity or numel == 0:
            self.overflowed += 1
            return torch.empty(shape, dtype=dtype, device=self.device)
        return block.narrow(0, start // size, numel).view(shape)
