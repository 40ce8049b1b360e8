"""The decode-attention entry point for callers that cannot allocate device memory.

Some host programs reach the kernels through the library's C symbols at a moment when they have no
allocator to call: a serving loop that must not stall on cudaMalloc, a process that has given all
device memory to another pool, a hook in which allocation is forbidden.  For them the library
exports ``b200_attention_decode_static``, which keeps the partial results of its key spans in an
array built into the library instead of in scratch memory the caller brings.

This test calls that symbol the way such a program would -- through ctypes, with raw pointers --
and checks it against the regular entry point on two calls in a row (the second with other inputs
and another span count, over whatever the first left in the array), and that a call too large for
the array is refused before anything runs.  It lives in a file of its own that pytest collects
last, and it passes alone in a fresh process as well as after all other tests."""
import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

ARGS = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
        c_int, c_void_p]


def _problem(seed, kv_lens, H, KVH, D):
    g = torch.Generator().manual_seed(seed)
    B = len(kv_lens)
    width = max(-(-n // 64) for n in kv_lens)
    n_pages = B * width
    table = torch.randperm(n_pages, generator=g).to(torch.int32).reshape(B, width)
    k_pool = torch.randn(n_pages, KVH, 64, D, generator=g).to(torch.bfloat16)
    v_pool = torch.randn(n_pages, KVH, D, 64, generator=g).to(torch.bfloat16)
    qkv = (torch.randn(B, (H + 2 * KVH) * D, generator=g) * 2).to(torch.bfloat16)
    return [t.cuda().contiguous() for t in (qkv, torch.tensor(kv_lens, dtype=torch.int32), table, k_pool, v_pool)]


def _plain(qkv, kv_lens, table, k_pool, v_pool, H, KVH, D):
    """The plain implementation's attention of each sequence's one query over its cached keys."""
    import plain_llama as P

    rows = []
    for i, n in enumerate(kv_lens):
        pages = table[i, : -(-n // 64)].long().cpu()
        k = k_pool.cpu().float()[pages].permute(0, 2, 1, 3).reshape(-1, KVH, D)[:n]        # [n, KVH, D]
        v = v_pool.cpu().float()[pages].permute(0, 3, 1, 2).reshape(-1, KVH, D)[:n]
        q = torch.zeros(n, H, D)
        q[-1] = qkv[i, : H * D].cpu().float().view(H, D)                                    # the query sits at the last position
        rows.append(P.causal_attention(q, k, v)[-1].reshape(H * D))
    return torch.stack(rows)


def test_entry_point_without_allocation_matches_the_regular_one():
    from gpullama3.java_b200.kernels import ops
    from gpullama3.java_b200.kernels.build import library

    lib = library("attention_decode")
    fn = lib.b200_attention_decode_static
    fn.argtypes, fn.restype = ARGS, c_int
    lib.b200_attention_decode_static_capacity.restype = c_longlong
    capacity = lib.b200_attention_decode_static_capacity()
    assert capacity == 2 * 1024 * 1024

    stream = torch.cuda.current_stream().cuda_stream
    for seed, kv_lens, (H, KVH, D), splits in [(1, [517, 64, 33, 300], (8, 2, 64), 4),
                                               (2, [100, 900, 5], (12, 4, 128), 7)]:
        qkv, lens, table, k_pool, v_pool = _problem(seed, kv_lens, H, KVH, D)
        B = len(kv_lens)
        want = torch.empty(B, H * D, dtype=torch.bfloat16, device="cuda")
        ops.attention_decode(qkv, qkv.shape[1], want, lens, table, k_pool, v_pool, H, KVH, D, 0, splits)
        got = torch.full_like(want, 7.0)
        # The lengths reach the device through a kernel that runs right before the call, as they would in a
        # serving loop that keeps them on the device: the entry point must not read them before that kernel is done.
        lens_late = torch.zeros_like(lens)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()      # the driver's own count: sees any cudaMalloc, not only torch's
        lens_late.add_(lens)
        status = fn(qkv.data_ptr(), qkv.shape[1], got.data_ptr(), lens_late.data_ptr(), table.data_ptr(), table.shape[1],
                    k_pool.data_ptr(), v_pool.data_ptr(), B, H, KVH, D, 0, splits, stream)
        torch.cuda.synchronize()
        assert status == 0
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.equal(got, want)                   # the same kernels on the same inputs: the same bits
        ref = _plain(qkv, kv_lens, table, k_pool, v_pool, H, KVH, D)
        scale = float(ref.abs().max())
        torch.testing.assert_close(got.float().cpu(), ref, rtol=2.0 ** -7, atol=2.0 ** -8 * scale)

    # Too large for the array: 64 sequences x 32 heads x 16 spans x (128 + 2) floats = 4.26 M floats.  The inputs
    # have the sizes the call names, so that a call wrongly let through would still stay inside them.
    qkv, lens, table, k_pool, v_pool = _problem(3, [40] * 64, 32, 8, 128)
    got = torch.zeros(64, 32 * 128, dtype=torch.bfloat16, device="cuda")
    status = fn(qkv.data_ptr(), qkv.shape[1], got.data_ptr(), lens.data_ptr(), table.data_ptr(), table.shape[1],
                k_pool.data_ptr(), v_pool.data_ptr(), 64, 32, 8, 128, 0, 16, stream)
    assert status == 10004
    # Misaligned queries (raw pointers come from anywhere): refused, not faulted on.
    status = fn(qkv.data_ptr() + 2, qkv.shape[1], got.data_ptr(), lens.data_ptr(), table.data_ptr(), table.shape[1],
                k_pool.data_ptr(), v_pool.data_ptr(), 63, 32, 8, 128, 0, 1, stream)
    assert status == 10002
    torch.cuda.synchronize()
