"""The fast attention kernels at the places where one key too many or too few hides in the noise of hundreds.

With random queries and keys a key that is wrongly dropped or wrongly read moves the output by about 1/n, below any
honest tolerance.  Here every query matches one chosen key far more strongly than all others, so the output is that
key's value if the key counts and something else entirely if it does not.  The chosen keys sit where kernels cut
their work: the query's own position and the one before it, the first key a window still reaches and the one it no
longer does, both sides of every 32-, 64- and 128-key boundary (span, page and block edges) and position 0.  Numbers
that are not finite, behind a sequence's end or in pages of other sequences, must not reach any output either."""
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def ops():
    from gpullama3.java_b200.kernels import ops as o
    return o


def _pages(n, KVH, D, seed, n_pages=None):
    """One sequence of ``n`` random keys and values in scattered pages; the rest of the pool (stale tails, pages
    of nobody) holds NaN keys and infinite values."""
    g = torch.Generator().manual_seed(seed)
    width = -(-n // 64)
    n_pages = n_pages or width + 3
    perm = torch.randperm(n_pages, generator=g)[:width]
    k = torch.randn(n, KVH, D, generator=g).to(BF).float()
    v = torch.randn(n, KVH, D, generator=g).to(BF).float()
    k_pool = torch.full((n_pages, KVH, 64, D), float("nan"))
    v_pool = torch.full((n_pages, KVH, D, 64), float("inf"))
    for lp in range(width):
        m = min(64, n - lp * 64)
        k_pool[perm[lp], :, :m] = k[lp * 64: lp * 64 + m].transpose(0, 1)
        v_pool[perm[lp], :, :, :m] = v[lp * 64: lp * 64 + m].permute(1, 2, 0)
    return k, v, k_pool.to(BF).cuda(), v_pool.to(BF).cuda(), perm.to(torch.int32)


def _hot_queries(k, targets, H):
    """Query i matches key targets[i] of its kv head: its score there is about 34 (strength * |k|^2 / sqrt(D)), the
    others are noise with a standard deviation of ``strength``."""
    KVH, D = k.shape[1], k.shape[2]
    strength = 34.0 / math.sqrt(D)
    q = torch.stack([k[t].repeat_interleave(H // KVH, dim=0) for t in targets]) * strength    # [n, H, D]
    return q.to(BF).float()


def _attend(q, k, v, pos, window):
    """inference/InferenceCore.java:106-145 for one query at position ``pos``: keys lo..pos, scores / sqrt(D),
    softmax, weighted values.  q [H, D]; k, v [n, KVH, D]."""
    H, D = q.shape
    KVH = k.shape[1]
    lo = max(0, pos + 1 - window) if window else 0
    out = torch.empty(H, D)
    for h in range(H):
        g = h // (H // KVH)
        s = (k[lo:pos + 1, g] @ q[h]) / math.sqrt(D)
        p = torch.exp(s - s.max())
        out[h] = (p / p.sum()) @ v[lo:pos + 1, g]
    return out


def _close(got, ref):
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, ref, rtol=2.0 ** -7, atol=2.0 ** -8 * float(ref.abs().max()))


@pytest.mark.parametrize("H, KVH, D", [(8, 2, 64), (4, 1, 128), (6, 3, 32), (3, 1, 96)])
@pytest.mark.parametrize("window", [0, 1, 33, 128, 200])
@pytest.mark.parametrize("n_splits", [1, 2, 3, 8, 16])
@pytest.mark.parametrize("fused", [False, True], ids=["attention_decode", "attention_decode_rope"])
def test_decode_attention_counts_every_key_once(H, KVH, D, window, n_splits, fused):
    """517 cached keys, 517 queries at the last position, query i matching key i: every key is some span's first,
    last or middle key, and with a window the keys before it are hot for queries that must not see them."""
    n = 517
    k, v, k_pool, v_pool, row = _pages(n, KVH, D, seed=D + H + window)
    q = _hot_queries(k, range(n), H)
    table = row[None, :].repeat(n, 1).cuda().contiguous()             # all queries read the same pages
    lens = torch.full((n,), n, dtype=torch.int32, device="cuda")
    qkv = torch.cat([q.reshape(n, H * D), torch.zeros(n, 2 * KVH * D)], dim=1).to(BF).cuda().contiguous()
    out = torch.full((n, H * D), 9.0, dtype=BF, device="cuda")
    if fused:    # no rotation (all frequencies zero) and nothing stored: the queries meet the cache as it is
        inv = torch.zeros(D // 2, dtype=torch.float32, device="cuda")
        ops().attention_decode_rope(qkv, out, lens, table, k_pool, v_pool, inv, H, KVH, D, 0, window, n_splits,
                                    write_cache=False)
    else:
        ops().attention_decode(qkv, qkv.shape[1], out, lens, table, k_pool, v_pool, H, KVH, D, window, n_splits)
    ref = torch.stack([_attend(q[i], k, v, n - 1, window) for i in range(n)]).reshape(n, H * D)
    lo = max(0, n - window) if window else 0
    # the premise: a query whose key counts gets that key's value (all but the few keys that happen to be short)
    hit = (ref.reshape(n, H, D)[lo:, 0] - v[lo:, 0]).abs().amax(dim=-1)
    assert float((hit < 0.1).float().mean()) > 0.9
    _close(out.float().cpu(), ref)


def _prefill_problem(H, KVH, D, window, n, q0, seed):
    """Sequences that share one set of pages; sequence j's query at position t matches the key its pattern names."""
    k, v, k_pool, v_pool, row = _pages(n, KVH, D, seed=seed)
    lo = (lambda t: max(0, t + 1 - window)) if window else (lambda t: 0)
    patterns = [lambda t: t, lambda t: max(0, t - 1), lambda t: lo(t), lambda t: max(0, lo(t) - 1),
                lambda t: (t // 128) * 128, lambda t: max(0, (t // 128) * 128 - 1), lambda t: (t // 64) * 64,
                lambda t: max(0, (t // 32) * 32 - 1), lambda t: 0, lambda t: t // 2]
    qs, refs, cu = [], [], [0]
    for pat in patterns:
        q = _hot_queries(k, [pat(t) for t in range(q0, n)], H)
        qs.append(q)
        refs.append(torch.stack([_attend(q[i], k, v, q0 + i, window) for i in range(n - q0)]))
        cu.append(cu[-1] + n - q0)
    B = len(patterns)
    q = torch.cat(qs).reshape(-1, H * D)
    qkv = torch.cat([q, torch.zeros(q.shape[0], 2 * KVH * D)], dim=1).to(BF).cuda().contiguous()
    table = row[None, :].repeat(B, 1).cuda().contiguous()
    lens = torch.full((B,), n, dtype=torch.int32, device="cuda")
    return qkv, torch.tensor(cu, dtype=torch.int32, device="cuda"), lens, table, k_pool, v_pool, \
        torch.cat(refs).reshape(-1, H * D), B


@pytest.mark.parametrize("H, KVH, D", [(4, 2, 64), (2, 1, 128), (6, 2, 32), (3, 1, 96)])
@pytest.mark.parametrize("window", [0, 1, 64, 129])
@pytest.mark.parametrize("n, q0", [(300, 0), (517, 130)])
def test_prefill_attention_counts_every_key_once(H, KVH, D, window, n, q0):
    """The kernel that reads keys and values straight into mma fragments (head sizes 32 to 128)."""
    qkv, cu, lens, table, k_pool, v_pool, ref, B = _prefill_problem(H, KVH, D, window, n, q0, seed=H + D + window)
    out = torch.full((qkv.shape[0], H * D), 9.0, dtype=BF, device="cuda")
    ops().attention_prefill(qkv, qkv.shape[1], out, cu, lens, table, k_pool, v_pool, B, n - q0, H, KVH, D, window)
    _close(out.float().cpu(), ref)


@pytest.mark.parametrize("H, KVH, D", [(4, 2, 64), (2, 1, 128), (3, 3, 64)])
@pytest.mark.parametrize("window", [0, 1, 64, 129])
@pytest.mark.parametrize("n, q0", [(300, 0), (517, 130), (700, 257)])
def test_tensor_memory_prefill_attention_counts_every_key_once(H, KVH, D, window, n, q0):
    """The tcgen05 kernel, one query tile at a time (windows, or little work)."""
    qkv, cu, lens, table, k_pool, v_pool, ref, B = _prefill_problem(H, KVH, D, window, n, q0, seed=H + D + window + 1)
    out = torch.full((qkv.shape[0], H * D), 9.0, dtype=BF, device="cuda")
    assert ops().attention_prefill_tc(qkv, qkv.shape[1], out, cu, lens, table, k_pool, v_pool, B, n - q0, H, KVH, D, window)
    assert ops().attention_prefill_tc_status() == 0
    _close(out.float().cpu(), ref)


@pytest.mark.parametrize("H, KVH, D", [(16, 4, 64), (16, 2, 128)])
@pytest.mark.parametrize("n, q0", [(700, 0), (900, 130)])
def test_tensor_memory_prefill_in_pairs_counts_every_key_once(H, KVH, D, n, q0):
    """The same kernel when it takes query tiles in pairs (no window, at least one unit of work per SM)."""
    qkv, cu, lens, table, k_pool, v_pool, ref, B = _prefill_problem(H, KVH, D, 0, n, q0, seed=H + D)
    assert -(-(n - q0) // 256) * H * B >= 148
    out = torch.full((qkv.shape[0], H * D), 9.0, dtype=BF, device="cuda")
    assert ops().attention_prefill_tc(qkv, qkv.shape[1], out, cu, lens, table, k_pool, v_pool, B, n - q0, H, KVH, D, 0)
    assert ops().attention_prefill_tc_status() == 0
    _close(out.float().cpu(), ref)
