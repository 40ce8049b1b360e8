"""The block of memory a pass takes its intermediate tensors from: a stack with marks, aligned pieces, growth
after a pass that did not fit."""
import pytest
import torch

from gpullama3.java_b200.engine.workspace import Workspace


def test_pieces_are_aligned_disjoint_and_given_back_in_stack_order():
    ws = Workspace("cpu", 64 * 1024)
    a = ws.take((3, 5), torch.float32)
    b = ws.take((7,), torch.bfloat16)
    assert a.shape == (3, 5) and a.dtype == torch.float32 and b.dtype == torch.bfloat16
    assert a.data_ptr() % 256 == 0 and b.data_ptr() % 256 == 0 and b.data_ptr() >= a.data_ptr() + 60
    a.fill_(1.0)
    b.fill_(2.0)
    assert float(a.sum()) == 15.0                      # writing one piece leaves the other alone
    mark = ws.mark()
    c = ws.take((100,), torch.float32)
    ws.release(mark)
    d = ws.take((50,), torch.int32)
    assert d.data_ptr() == c.data_ptr()                # the same memory again after the release
    ws.release(0)
    with pytest.raises(ValueError):
        ws.release(10)                                 # beyond what is taken
    assert ws.overflowed == 0


def test_a_pass_that_does_not_fit_is_served_and_the_block_grows_for_the_next():
    ws = Workspace("cpu")                               # starts empty
    x = ws.take((1000,), torch.float32)
    y = ws.take((10, 10), torch.float32)
    assert x.numel() == 1000 and y.shape == (10, 10) and ws.overflowed == 2
    ws.reset()
    assert ws.capacity >= 4000 + 400
    z = ws.take((1000,), torch.float32)
    assert ws.overflowed == 2 and z.data_ptr() % 256 == 0
    ws.reset()
    big = ws.take((ws.capacity,), torch.float32)        # four times the block: from the allocator this once
    assert big.numel() == ws.capacity and ws.overflowed == 3
    assert ws.take((0, 4), torch.float32).numel() == 0
