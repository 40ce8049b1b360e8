"""Each CUDA kernel alone against its plain formula, at sizes other than the tiny models': widths
and vocabularies that are no power of two, head sizes in steps of 16, odd head counts and groups,
scattered cache pages, windows."""
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, ref=None):
    """float32: accumulation-order noise, 2e-5 of the largest value.  bfloat16 (inputs already
    rounded, the reference rounded at the end): two units in the last place of each value."""
    scale = float(ref.abs().max()) if ref is not None else 1.0
    if dtype == torch.float32:
        return dict(rtol=0.0, atol=2e-5 * scale)
    return dict(rtol=2.0 ** -7, atol=2e-5 * scale)


def ops():
    from gpullama3.java_b200.kernels import ops as o
    return o


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab, dim", [(37, 24), (1000, 1030)])
def test_embed_gather(dtype, vocab, dim):
    table = torch.randn(vocab, dim, device="cuda").to(dtype)
    tokens = torch.randint(0, vocab, (19,), device="cuda", dtype=torch.int32)
    out = torch.empty(19, dim, device="cuda")
    ops().embed_gather(table, tokens, out)
    assert torch.equal(out, table.float()[tokens.long()])


@pytest.mark.parametrize("w_dtype", DTYPES)
@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("dim, eps", [(24, 1e-5), (1030, 1e-6), (4096, 1e-2)])
def test_rmsnorm(w_dtype, out_dtype, dim, eps):
    x = torch.randn(7, dim, device="cuda") * 3
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(w_dtype)
    out = torch.empty(7, dim, device="cuda", dtype=out_dtype)
    ops().rmsnorm(x, w, out, eps)
    ref = P.rmsnorm(x.cpu(), w.float().cpu(), eps)
    torch.testing.assert_close(out.float().cpu(), ref.to(out_dtype).float(), **tol(out_dtype, ref))
    rows = torch.tensor([5, 0, 5], device="cuda", dtype=torch.int32)
    out2 = torch.empty(3, dim, device="cuda", dtype=out_dtype)
    ops().rmsnorm(x, w, out2, eps, rows)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("w_dtype", DTYPES)
@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("n_rows, dim", [(1024, 1024), (1027, 2048), (1500, 3072), (1030, 4096), (1024, 5120)])
def test_rmsnorm_of_many_rows(w_dtype, out_dtype, n_rows, dim):
    """A prompt's worth of rows takes the warp-per-row kernel at the usual widths (1024-wide steps up to 4096; 5120
    does not): a count of rows that does not fill the last CTA, each row with a scale of its own, and a selection."""
    g = torch.Generator().manual_seed(n_rows + dim)
    x = (torch.randn(n_rows, dim, generator=g) * (0.1 + 5 * torch.rand(n_rows, 1, generator=g))).cuda()
    w = (1 + 0.1 * torch.randn(dim, generator=g)).cuda().to(w_dtype)
    out = torch.full((n_rows, dim), 7.0, device="cuda", dtype=out_dtype)
    ops().rmsnorm(x, w, out, 1e-5)
    ref = P.rmsnorm(x.cpu(), w.float().cpu(), 1e-5)
    torch.testing.assert_close(out.float().cpu(), ref.to(out_dtype).float(), **tol(out_dtype, ref))
    rows = torch.randperm(n_rows, generator=g)[:1024].to(torch.int32).cuda()
    out2 = torch.empty(1024, dim, device="cuda", dtype=out_dtype)
    ops().rmsnorm(x, w, out2, 1e-5, rows)
    assert torch.equal(out2, out[rows.long()])


def _paged_setup(dtype, n_seqs, kv_lens, KVH, D, n_pages, seed=0):
    """Random keys/values laid out in scattered pages; returns pools, the page table and the dense
    per-sequence keys/values."""
    g = torch.Generator().manual_seed(seed)
    width = max(-(-n // 64) for n in kv_lens)
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(n_seqs, width, dtype=torch.int32)
    k_pool = torch.zeros(n_pages, KVH, 64, D)
    v_pool = torch.zeros(n_pages, KVH, D, 64)
    dense = []
    for s, n in enumerate(kv_lens):
        k = torch.randn(n, KVH, D, generator=g).to(dtype).float()
        v = torch.randn(n, KVH, D, generator=g).to(dtype).float()
        dense.append((k, v))
        for lp in range(-(-n // 64)):
            page = perm.pop()
            table[s, lp] = page
            m = min(64, n - lp * 64)
            k_pool[page, :, :m] = k[lp * 64:lp * 64 + m].transpose(0, 1)
            v_pool[page, :, :, :m] = v[lp * 64:lp * 64 + m].permute(1, 2, 0)
    return k_pool.to(dtype).cuda(), v_pool.to(dtype).cuda(), table.cuda(), dense


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, KVH, D, window", [(4, 2, 16, 0), (3, 1, 32, 0), (6, 3, 48, 0), (8, 8, 64, 0),
                                               (5, 5, 80, 0), (8, 2, 128, 0), (2, 1, 256, 0), (4, 1, 64, 37),
                                               (4, 2, 32, 200)])
def test_attention_paged_against_plain(dtype, H, KVH, D, window):
    """Queries of several sequences at scattered positions (chunks continuing a prefix and single
    decoded tokens together) over scattered pages."""
    kv_lens = [1, 64, 65, 300, 129]
    q_starts = [0, 60, 64, 299, 100]   # each sequence's queries cover positions q_start .. kv_len-1
    k_pool, v_pool, table, dense = _paged_setup(dtype, len(kv_lens), kv_lens, KVH, D, n_pages=40, seed=D + H)
    g = torch.Generator().manual_seed(1)
    qs, positions, seq_ids, refs = [], [], [], []
    for s, (n, q0) in enumerate(zip(kv_lens, q_starts)):
        k, v = dense[s]
        q_full = (torch.randn(n, H, D, generator=g) * 2).to(dtype).float()
        ref_full = P.causal_attention(q_full, k, v, window or None)
        qs.append(q_full[q0:])
        refs.append(ref_full[q0:])
        positions += list(range(q0, n))
        seq_ids += [s] * (n - q0)
    q = torch.cat(qs).reshape(-1, H * D)
    # queries sit at the start of wider rows, as in the fused qkv buffer
    qkv = torch.cat([q, torch.randn(q.shape[0], 2 * KVH * D)], dim=1).to(dtype).cuda().contiguous()
    out = torch.empty(q.shape[0], H * D, dtype=dtype, device="cuda")
    pos_t = torch.tensor(positions, dtype=torch.int32, device="cuda")
    seq_t = torch.tensor(seq_ids, dtype=torch.int32, device="cuda")
    ops().attention_paged(qkv, qkv.shape[1], out, pos_t, seq_t, table, k_pool, v_pool, H, KVH, D, window)
    ref = torch.cat(refs).reshape(-1, H * D)
    torch.testing.assert_close(out.float().cpu(), ref.to(dtype).float(), **tol(dtype, ref))
    # the keys of every token cut into spans (more spans than some tokens have tiles of keys: empty spans)
    for n_splits in (2, 5):
        cut = torch.full_like(out, 7.0)
        ops().attention_paged(qkv, qkv.shape[1], cut, pos_t, seq_t, table, k_pool, v_pool, H, KVH, D, window, n_splits=n_splits)
        torch.testing.assert_close(cut.float().cpu(), ref.to(dtype).float(), **tol(dtype, ref))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """One key far back matches the query strongly: the output must be that key's value."""
    H, KVH, D, n = 2, 1, 32, 700
    k_pool, v_pool, table, dense = _paged_setup(dtype, 1, [n], KVH, D, n_pages=16, seed=9)
    k, v = dense[0]
    target = 123
    q = (k[target, 0] * 6.0).repeat(H).reshape(1, H * D)      # score ~ 6 |k|^2 / sqrt(D), far above the rest
    qkv = torch.cat([q, torch.zeros(1, 2 * KVH * D)], dim=1).to(dtype).cuda()
    out = torch.empty(1, H * D, dtype=dtype, device="cuda")
    ops().attention_paged(qkv, qkv.shape[1], out, torch.tensor([n - 1], dtype=torch.int32, device="cuda"),
                          torch.tensor([0], dtype=torch.int32, device="cuda"), table, k_pool, v_pool, H, KVH, D, 0)
    ref = P.causal_attention(q.to(dtype).float().reshape(1, H, D).expand(n, H, D).contiguous(), k, v)[-1]
    torch.testing.assert_close(out.float().cpu().reshape(H, D), ref.to(dtype).float(), **tol(dtype, ref))
    assert float((out.float().cpu().reshape(H, D)[0] - v[target, 0]).abs().max()) < 0.05
    cut = torch.empty_like(out)                               # the far key lies in the first of four spans
    ops().attention_paged(qkv, qkv.shape[1], cut, torch.tensor([n - 1], dtype=torch.int32, device="cuda"),
                          torch.tensor([0], dtype=torch.int32, device="cuda"), table, k_pool, v_pool, H, KVH, D, 0, n_splits=4)
    assert float((cut.float().cpu().reshape(H, D)[0] - v[target, 0]).abs().max()) < 0.05


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairing", ["interleaved", "half"])
@pytest.mark.parametrize("H, KVH, D, rotary", [(4, 2, 16, 16), (3, 1, 32, 32), (2, 2, 48, 32), (1, 1, 128, 0)])
def test_rope_and_cache_write(dtype, pairing, H, KVH, D, rotary):
    from gpullama3.java_b200.parts.position import PAIRING_CODES

    positions = [0, 1, 63, 64, 65, 200, 4095, 7]
    seq_ids = [0, 0, 0, 0, 0, 0, 1, 1]
    T = len(positions)
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(T, (H + 2 * KVH) * D, generator=g).to(dtype)
    scaling = {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 32}
    inv = P.rope_inverse_frequencies(rotary, 5e5, scaling) if rotary else torch.zeros(1, dtype=torch.float64)
    n_pages = 70
    table = torch.zeros(2, 64, dtype=torch.int32)
    table[0] = torch.arange(64)[torch.randperm(64, generator=g)][:64]
    table[1, 63] = 65
    table[1, 0] = 66
    k_pool = torch.zeros(n_pages, KVH, 64, D, dtype=dtype, device="cuda")
    v_pool = torch.zeros(n_pages, KVH, D, 64, dtype=dtype, device="cuda")
    buf = qkv.clone().cuda()
    ops().rope_cache_write(buf, torch.tensor(positions, dtype=torch.int32, device="cuda"),
                           torch.tensor(seq_ids, dtype=torch.int32, device="cuda"), table.cuda(),
                           inv.to(torch.float32).cuda(), k_pool, v_pool, H, KVH, D, rotary, PAIRING_CODES[pairing])
    x = qkv.float()
    q, k, v = x[:, :H * D].reshape(T, H, D), x[:, H * D:(H + KVH) * D].reshape(T, KVH, D), x[:, (H + KVH) * D:].reshape(T, KVH, D)
    if rotary:
        cos, sin = P.rope_tables(torch.tensor(positions), inv, torch.float32)
        q = torch.cat([P.apply_rope(q[..., :rotary], cos, sin, pairing), q[..., rotary:]], dim=-1)
        k = torch.cat([P.apply_rope(k[..., :rotary], cos, sin, pairing), k[..., rotary:]], dim=-1)
    t = tol(dtype, x)
    torch.testing.assert_close(buf[:, :H * D].float().cpu(), q.reshape(T, H * D).to(dtype).float(), **t)
    for i, (p, s) in enumerate(zip(positions, seq_ids)):
        page = int(table[s, p // 64])
        torch.testing.assert_close(k_pool[page, :, p % 64].float().cpu(), k[i].to(dtype).float(), **t)
        assert torch.equal(v_pool[page, :, :, p % 64].float().cpu(), v[i])
    assert int((k_pool.float().abs().sum(dim=(1, 3)) > 0).sum()) == T   # no other cache row was touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairing, H, KVH, D", [("half", 8, 2, 64), ("interleaved", 3, 1, 96), ("half", 4, 4, 128),
                                                ("interleaved", 6, 2, 32)])
def test_rope_and_cache_write_for_prompts(dtype, pairing, H, KVH, D):
    """Many tokens go through the kernel that takes 16 tokens per CTA: a prompt from position 0 (tiles that lie
    aligned in their pages), a prompt whose tokens start at an odd offset of the batch, a chunk that continues at
    position 101 and crosses pages, a single token, and a last tile that is not full."""
    from gpullama3.java_b200.parts.position import PAIRING_CODES

    runs = [(0, 0, 200), (1, 0, 77), (2, 101, 150), (3, 4000, 1), (1, 77, 30)]   # (sequence, first position, tokens)
    positions = [p0 + i for _, p0, n in runs for i in range(n)]
    seq_ids = [s for s, _, n in runs for _ in range(n)]
    T = len(positions)
    assert T >= 64 and T % 16 != 0
    g = torch.Generator().manual_seed(8)
    qkv = torch.randn(T, (H + 2 * KVH) * D, generator=g).to(dtype)
    inv = P.rope_inverse_frequencies(D, 5e5, None)
    n_pages = 4 * 64
    table = torch.randperm(n_pages, generator=g).to(torch.int32).reshape(4, 64)
    k_pool = torch.zeros(n_pages, KVH, 64, D, dtype=dtype, device="cuda")
    v_pool = torch.zeros(n_pages, KVH, D, 64, dtype=dtype, device="cuda")
    buf = qkv.clone().cuda()
    ops().rope_cache_write(buf, torch.tensor(positions, dtype=torch.int32, device="cuda"),
                           torch.tensor(seq_ids, dtype=torch.int32, device="cuda"), table.cuda(),
                           inv.to(torch.float32).cuda(), k_pool, v_pool, H, KVH, D, D, PAIRING_CODES[pairing])
    x = qkv.float()
    q, k, v = x[:, :H * D].reshape(T, H, D), x[:, H * D:(H + KVH) * D].reshape(T, KVH, D), x[:, (H + KVH) * D:].reshape(T, KVH, D)
    cos, sin = P.rope_tables(torch.tensor(positions), inv, torch.float32)
    q, k = P.apply_rope(q, cos, sin, pairing), P.apply_rope(k, cos, sin, pairing)
    t = tol(dtype, x)
    torch.testing.assert_close(buf[:, :H * D].float().cpu(), q.reshape(T, H * D).to(dtype).float(), **t)
    assert torch.equal(buf[:, H * D:].cpu(), qkv[:, H * D:])          # raw keys and values stay as they were
    pages = table[torch.tensor(seq_ids), torch.tensor(positions) // 64].long()
    slots = torch.tensor(positions) % 64
    torch.testing.assert_close(k_pool.cpu()[pages, :, slots].float(), k.to(dtype).float(), **t)
    assert torch.equal(v_pool.cpu()[pages, :, :, slots].float(), v)
    assert int((k_pool.float().abs().sum(dim=(1, 3)) > 0).sum()) == T   # no other cache row was touched
    assert int((v_pool.float().abs().sum(dim=(1, 2)) > 0).sum()) == T


@pytest.mark.parametrize("a_dtype, w_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                              (torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M, N, K", [(1, 40, 24), (7, 130, 100), (65, 64, 17), (200, 258, 1030),
                                     (16, 1002, 2048), (9, 36, 8192), (3, 50, 1022), (17, 30, 64)])
def test_gemm_generic_and_its_epilogues(a_dtype, w_dtype, M, N, K):
    """The plain product in its two forms: at most 16 rows with rows that start on 4-element boundaries stream the
    weights (a last CTA with one pair of rows, K of one pass per lane and of sixty-four); everything else is tiled."""
    o = ops()
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(a_dtype).cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(w_dtype).cuda()
    ref = a.float().cpu().double() @ w.float().cpu().double().t()
    c = torch.empty(M, N, dtype=a_dtype, device="cuda")
    o.gemm_generic(a, w, c, o.EPILOGUE_STORE)
    torch.testing.assert_close(c.float().cpu(), ref.float().to(a_dtype).float(), **tol(a_dtype, ref))
    res0 = torch.randn(M, N, generator=g)
    res = res0.clone().cuda()
    o.gemm_generic(a, w, res, o.EPILOGUE_RESIDUAL_ADD)
    torch.testing.assert_close(res.cpu(), (res0.double() + ref).float(), **tol(torch.float32, ref))
    h = torch.empty(M, N // 2, dtype=a_dtype, device="cuda")
    o.gemm_generic(a, w, h, o.EPILOGUE_GATED_SILU)
    gated = P.swiglu(ref[:, 0::2], ref[:, 1::2])
    torch.testing.assert_close(h.float().cpu(), gated.float().to(a_dtype).float(), **tol(a_dtype, gated))


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 32, 50, 64])
@pytest.mark.parametrize("N, K", [(16, 32), (50, 96), (200, 2048), (4098, 64), (5000, 1056), (2400, 1088)])
def test_gemm_decode_and_its_epilogues(M, N, K):
    # (2400 x 1088: the grid of up to three CTAs per SM whose rounds are six k-blocks, ending inside a round)
    o = ops()
    g = torch.Generator().manual_seed(M * N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).cuda()
    ref = a.float().cpu().double() @ w.float().cpu().double().t()
    for c_dtype in (torch.bfloat16, torch.float32):
        c = torch.full((M, N), 7.0, dtype=c_dtype, device="cuda")
        assert o.gemm_decode(a, w, c, o.EPILOGUE_STORE)
        torch.testing.assert_close(c.float().cpu(), ref.float().to(c_dtype).float(), **tol(c_dtype, ref))
    res0 = torch.randn(M, N, generator=g)
    res = res0.clone().cuda()
    assert o.gemm_decode(a, w, res, o.EPILOGUE_RESIDUAL_ADD)
    torch.testing.assert_close(res.cpu(), (res0.double() + ref).float(), **tol(torch.float32, ref))
    h = torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda")
    assert o.gemm_decode(a, w, h, o.EPILOGUE_GATED_SILU)
    gated = P.swiglu(ref[:, 0::2], ref[:, 1::2])
    torch.testing.assert_close(h.float().cpu(), gated.float().to(torch.bfloat16).float(), **tol(torch.bfloat16, gated))
    # a strided view of a wider buffer, and shapes the kernel leaves to the plain one
    wide = torch.randn(M, K + 64, generator=g).to(torch.bfloat16).cuda()
    c = torch.empty(M, N, dtype=torch.float32, device="cuda")
    assert o.gemm_decode(wide[:, :K], w, c)
    torch.testing.assert_close(c.cpu(), (wide[:, :K].float().cpu().double() @ w.float().cpu().double().t()).float(),
                               **tol(torch.float32, ref))
    assert not o.gemm_decode(torch.zeros(65, K, dtype=torch.bfloat16, device="cuda"), w, c)
    assert not o.gemm_decode(a.float(), w, c)


@pytest.mark.parametrize("M", [1, 8, 13, 16])
@pytest.mark.parametrize("hidden, K, N2", [(544, 96, 96), (2400, 64, 50), (4128, 32, 40)])
@pytest.mark.parametrize("w_dtype", [torch.bfloat16, torch.float32], ids=["w16", "w32"])
def test_gemm_decode_halves_of_a_split_norm(M, hidden, K, N2, w_dtype):
    """RMSNorm between two products without a kernel of its own: the residual product also leaves x * w and
    per-CTA sums of x^2 (68, 300 and 258 partial sums per row here: under and over the 256 a warp asks for
    up front, 8 and 16 rows per CTA), the next product applies rsqrt(mean(x^2) + eps) to its sums.  Checked
    half by half and end to end against the norm followed by the product."""
    o = ops()
    eps = 1e-5
    g = torch.Generator().manual_seed(M + hidden)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w1 = (torch.randn(hidden, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).cuda()
    x0 = torch.randn(M, hidden, generator=g)
    nw = (1.0 + 0.2 * torch.randn(hidden, generator=g)).to(w_dtype)
    x_ref = x0.double() + a.float().cpu().double() @ w1.float().cpu().double().t()
    res = x0.clone().cuda()
    act = torch.empty(M, hidden, dtype=torch.bfloat16, device="cuda")
    P_out = o.gemm_decode_partials(M, hidden)
    assert P_out == {544: 68, 2400: 300, 4128: 258}[hidden]
    partials = torch.full((M, P_out), 99.0, device="cuda")
    o.gemm_decode_linked(a, w1, res, o.EPILOGUE_RESIDUAL_ADD, emit=(nw.cuda(), act, partials))
    torch.testing.assert_close(res.cpu(), x_ref.float(), **tol(torch.float32, x_ref))
    x = res.cpu().double()                                            # what the kernel itself holds
    torch.testing.assert_close(act.float().cpu(), (x * nw.double()).float().to(torch.bfloat16).float(), rtol=2.0 ** -7, atol=1e-6)
    torch.testing.assert_close(partials.sum(dim=1).cpu().double(), (x * x).sum(dim=1), rtol=1e-5, atol=0)
    # second half against what it is given: act (already rounded) and the factor of the partial sums
    w2 = (torch.randn(N2, hidden, generator=g) / math.sqrt(hidden)).to(torch.bfloat16).cuda()
    r = torch.rsqrt(partials.sum(dim=1).cpu().double() / hidden + eps).reshape(M, 1)
    want = (act.float().cpu().double() @ w2.float().cpu().double().t()) * r
    for c_dtype in (torch.bfloat16, torch.float32):
        c = torch.empty(M, N2, dtype=c_dtype, device="cuda")
        o.gemm_decode_linked(act, w2, c, o.EPILOGUE_STORE, row_factors=(partials, eps, hidden))
        torch.testing.assert_close(c.float().cpu(), want.float().to(c_dtype).float(), **tol(c_dtype, want))
    h = torch.empty(M, N2 // 2, dtype=torch.bfloat16, device="cuda")
    o.gemm_decode_linked(act, w2, h, o.EPILOGUE_GATED_SILU, row_factors=(partials, eps, hidden))
    gated = P.swiglu(want[:, 0::2], want[:, 1::2])
    torch.testing.assert_close(h.float().cpu(), gated.float().to(torch.bfloat16).float(), **tol(torch.bfloat16, gated))
    # and against the norm as a kernel of its own followed by the product.  Both ways round the product's input to
    # bfloat16 once, at different places (x w r against x w): per term a relative 2^-9 at most, so two sums of
    # `hidden` such terms differ by about 2^-9 of the result's size; 2^-7 of the largest result bounds 96 of them
    normed = torch.empty(M, hidden, dtype=torch.bfloat16, device="cuda")
    o.rmsnorm(res, nw.cuda(), normed, eps)
    apart = torch.empty(M, N2, dtype=torch.float32, device="cuda")
    assert o.gemm_decode(normed, w2, apart, o.EPILOGUE_STORE)
    assert float((c.float() - apart).abs().max()) <= 2.0 ** -7 * float(apart.abs().max())
    exact = P.rmsnorm(x.float(), nw.float(), eps).double() @ w2.float().cpu().double().t()
    assert float((c.float().cpu() - exact).abs().max()) <= 2.0 ** -7 * float(exact.abs().max())
    # both halves in one call: the residual product of a second layer
    res2 = torch.zeros(M, N2, device="cuda")
    act2 = torch.empty(M, N2, dtype=torch.bfloat16, device="cuda")
    part2 = torch.empty(M, o.gemm_decode_partials(M, N2), device="cuda")
    o.gemm_decode_linked(act, w2, res2, o.EPILOGUE_RESIDUAL_ADD, row_factors=(partials, eps, hidden),
                         emit=(torch.ones(N2, dtype=w_dtype, device="cuda"), act2, part2))
    torch.testing.assert_close(res2.cpu(), want.float(), **tol(torch.bfloat16, want))
    torch.testing.assert_close(part2.sum(dim=1).cpu().double(), (res2.cpu().double() ** 2).sum(dim=1), rtol=1e-5, atol=0)


def _check_gemm_tcgen05(gemm, M, N, K):
    """Store (both output types), residual add and gated SiLU of ``gemm`` against the plain product."""
    o = ops()
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).cuda()
    ref = a.float().cpu().double() @ w.float().cpu().double().t()
    for c_dtype in (torch.bfloat16, torch.float32):
        c = torch.full((M, N), 7.0, dtype=c_dtype, device="cuda")
        assert gemm(a, w, c, o.EPILOGUE_STORE)
        torch.testing.assert_close(c.float().cpu(), ref.float().to(c_dtype).float(), **tol(c_dtype, ref))
    res0 = torch.randn(M, N, generator=g)
    res = res0.clone().cuda()
    assert gemm(a, w, res, o.EPILOGUE_RESIDUAL_ADD)
    torch.testing.assert_close(res.cpu(), (res0.double() + ref).float(), **tol(torch.float32, ref))
    if N % 2 == 0:
        h = torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda")
        assert gemm(a, w, h, o.EPILOGUE_GATED_SILU)
        gated = P.swiglu(ref[:, 0::2], ref[:, 1::2])
        torch.testing.assert_close(h.float().cpu(), gated.float().to(torch.bfloat16).float(), **tol(torch.bfloat16, gated))
    assert o.gemm_tcgen05_status() == 0
    return a, w


@pytest.mark.parametrize("M, N, K", [(128, 256, 64), (128, 256, 512), (1, 8, 8), (100, 300, 72), (129, 257, 200),
                                     (300, 1030, 2048), (2048, 512, 1024), (65, 3072, 2048)])
@pytest.mark.parametrize("width", [0, 256, 128, 64])
def test_gemm_tcgen05_and_its_epilogues(M, N, K, width):
    """The TMA + tcgen05 kernel at tile-exact sizes, at ragged edges in M, N and K, and with several
    waves of tiles, for each width of tile and for the choice the shape makes (0); every internal wait must
    have completed (status word 0)."""
    import functools
    o = ops()
    a, w = _check_gemm_tcgen05(functools.partial(o.gemm_tcgen05, tile_width=width), M, N, K)
    assert not o.gemm_tcgen05(a.float(), w, torch.empty(M, N, device="cuda"))
    if K % 16 == 8:   # a view whose rows are not 16-byte aligned is left to the plain kernel
        assert not o.gemm_tcgen05(a[:, 4:], w[:, 4:], torch.empty(M, N, device="cuda"))


@pytest.mark.parametrize("M, N, K", [(256, 256, 64), (256, 256, 512), (1, 8, 8), (100, 300, 72), (129, 257, 200), (257, 130, 136),
                                     (300, 1030, 2048), (2048, 512, 1024), (2048, 3072, 2048), (1000, 20000, 256)])
@pytest.mark.parametrize("width", [256, 128])
def test_gemm_tcgen05_by_pairs_of_ctas(M, N, K, width):
    """Tiles of 256 rows computed by two CTAs that each load their rows of the activations and half of the weight
    stage: exact tiles, ragged edges (a second CTA with few rows, or none; a half of the weight stage beyond N),
    several waves of tiles, more k-steps than stages, every epilogue.  Run twice: the same bits."""
    import functools
    o = ops()
    a, w = _check_gemm_tcgen05(functools.partial(o.gemm_tcgen05, tile_width=width, cta_pair=1), M, N, K)
    c1 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    c2 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    assert o.gemm_tcgen05(a, w, c1, tile_width=width, cta_pair=1) and o.gemm_tcgen05(a, w, c2, tile_width=width, cta_pair=-1)
    assert torch.equal(c1, c2)      # the same sums in the same order as the single-CTA kernel
    assert o.gemm_tcgen05_status() == 0


@pytest.mark.parametrize("H, KVH, D, M, K", [(32, 8, 64, 1300, 512), (32, 8, 64, 900, 512), (8, 2, 128, 2100, 256),
                                            (24, 8, 128, 700, 384), (5, 1, 64, 6500, 64)])
@pytest.mark.parametrize("pairing", [0, 1], ids=["interleaved", "half"])
@pytest.mark.parametrize("write_cache", [True, False], ids=["writes", "reads_only"])
def test_projection_with_rotation_and_cache_write_in_its_epilogue(H, KVH, D, M, K, pairing, write_cache):
    """The query/key/value product that rotates and writes the cache itself against the product followed by the rotation
    kernel: the same bits in the queries and in every page, nothing else touched.  Three sequences packed into one
    pass, one of them continuing at a position that is no multiple of anything, pages scattered; shapes that take
    the pairs of CTAs and shapes that take single CTAs; both pairings; a layer that only reads the cache."""
    o = ops()
    g = torch.Generator().manual_seed(H * D + M + pairing)
    N = (H + 2 * KVH) * D
    lens = [M // 2, M // 3, M - M // 2 - M // 3]
    starts = [0, 77, 0]
    positions = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(torch.int32).cuda()
    seq_ids = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).to(torch.int32).cuda()
    width = max(-(-(s + n) // 64) for s, n in zip(starts, lens))
    n_pages = 3 * width + 5
    table = torch.randperm(n_pages, generator=g)[:3 * width].to(torch.int32).reshape(3, width).cuda()
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).cuda()
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))).cuda()
    k0 = torch.randn(n_pages, KVH, 64, D, generator=g).to(torch.bfloat16).cuda()
    v0 = torch.randn(n_pages, KVH, D, 64, generator=g).to(torch.bfloat16).cuda()
    # the two kernels one after the other
    qkv_ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    assert o.gemm_tcgen05(a, w, qkv_ref, o.EPILOGUE_STORE)
    k_ref, v_ref = k0.clone(), v0.clone()
    o.rope_cache_write(qkv_ref, positions, seq_ids, table, inv_freq, k_ref if write_cache else None,
                       v_ref if write_cache else None, H, KVH, D, D, pairing, write_cache=write_cache)
    # the one product
    angles = o.rope_angles(positions, inv_freq, D // 2)
    ref_angle = positions.cpu().float()[:, None] * inv_freq.cpu()[None, :]
    torch.testing.assert_close(angles[..., 0].cpu().t(), torch.cos(ref_angle), rtol=0, atol=2e-6)
    torch.testing.assert_close(angles[..., 1].cpu().t(), torch.sin(ref_angle), rtol=0, atol=2e-6)
    qkv = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    k_got, v_got = k0.clone(), v0.clone()
    assert o.gemm_tcgen05_qkv_rope(a, w, qkv, positions, seq_ids, table, angles, k_got if write_cache else None,
                                   v_got if write_cache else None, H, KVH, D, pairing, write_cache)
    assert o.gemm_tcgen05_status() == 0
    assert torch.equal(qkv[:, :H * D], qkv_ref[:, :H * D])
    assert torch.equal(k_got, k_ref) and torch.equal(v_got, v_ref)
    assert bool((qkv[:, H * D:] == 7.0).all())          # key and value columns of the projection buffer are not written
    if write_cache:                                     # and the pages hold what the plain formulas give
        kv = (a.float().cpu().double() @ w.float().cpu().double().t()).float().to(torch.bfloat16).float()
        i = M // 2 + 5                                  # a token of the continuing sequence
        pos, page = int(positions[i]), int(table[1, int(positions[i]) // 64])
        want_v = kv[i, (H + KVH) * D:].view(KVH, D)
        torch.testing.assert_close(v_got[page, :, :, pos % 64].float().cpu(), want_v, rtol=2.0 ** -7, atol=2.0 ** -7)
        cs, sn = torch.cos(ref_angle[i]), torch.sin(ref_angle[i])
        kk = kv[i, H * D:(H + KVH) * D].view(KVH, D)
        x0, x1 = (kk[:, 0::2], kk[:, 1::2]) if pairing == 0 else (kk[:, :D // 2], kk[:, D // 2:])
        r0, r1 = x0 * cs - x1 * sn, x0 * sn + x1 * cs
        want_k = torch.stack([r0, r1], dim=-1).reshape(KVH, D) if pairing == 0 else torch.cat([r0, r1], dim=-1)
        torch.testing.assert_close(k_got[page, :, pos % 64, :].float().cpu(), want_k, rtol=2.0 ** -6, atol=2.0 ** -6)


def test_projection_with_rotation_declines_what_it_does_not_take():
    o = ops()
    H, KVH, K = 4, 2, 64
    for D, M in [(32, 3000), (64, 40), (96, 3000)]:
        N = (H + 2 * KVH) * D
        a = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda")
        w = torch.zeros(N, K, dtype=torch.bfloat16, device="cuda")
        qkv = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        pos = torch.arange(M, dtype=torch.int32, device="cuda")
        table = torch.arange(-(-M // 64), dtype=torch.int32, device="cuda").reshape(1, -1)
        angles = torch.zeros(D // 2, M, 2, device="cuda")
        kp = torch.zeros(table.numel(), KVH, 64, D, dtype=torch.bfloat16, device="cuda")
        vp = torch.zeros(table.numel(), KVH, D, 64, dtype=torch.bfloat16, device="cuda")
        assert not o.gemm_tcgen05_qkv_rope(a, w, qkv, pos, torch.zeros_like(pos), table, angles, kp, vp, H, KVH, D, 0, True)


@pytest.mark.parametrize("M, N, K, spans", [(128, 128, 128, 2), (100, 300, 328, 4), (300, 1030, 2048, 2), (256, 2048, 8192, 4),
                                            (129, 130, 320, 4), (512, 2048, 8192, 0), (256, 1024, 4096, 0)])
def test_gemm_tcgen05_with_k_cut_among_a_cluster(M, N, K, spans):
    """K cut into 2 or 4 spans whose partial tiles meet through distributed shared memory: exact tiles, ragged
    edges, a K whose last span is short or empty (328 = 6 k-steps over 4 spans: 2, 2, 2, 0; 320: 2, 2, 1, 0), and
    the shapes (few tiles, long K) for which the kernel is chosen without being asked.  Run twice: the sum must
    not depend on timing."""
    import functools
    o = ops()
    a, w = _check_gemm_tcgen05(functools.partial(o.gemm_tcgen05, k_spans=spans), M, N, K)
    c1 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    c2 = torch.empty(M, N, dtype=torch.float32, device="cuda")
    assert o.gemm_tcgen05(a, w, c1, k_spans=spans) and o.gemm_tcgen05(a, w, c2, k_spans=spans)
    assert torch.equal(c1, c2)
    if spans == 0:
        assert o.gemm_tcgen05_k_spans(M, N, K) == {512: 2, 256: 4}[M]
    assert o.gemm_tcgen05_status() == 0


@pytest.mark.parametrize("M", [1, 17, 32, 33, 64, 100, 128])
@pytest.mark.parametrize("N, K, splits", [(128, 64, None), (300, 200, None), (2048, 2048, None), (2048, 2048, 1),
                                          (130, 1024, 5), (16384, 512, None), (258, 8192, 8), (2048, 8192, 3)])
def test_gemm_skinny_and_its_epilogues(M, N, K, splits):
    """Few tokens against many weight rows, with K cut into spans whose partial tiles a cluster of CTAs
    adds up through distributed shared memory; the same inputs twice must give the same bits."""
    o = ops()
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).cuda()
    ref = a.float().cpu().double() @ w.float().cpu().double().t()
    for c_dtype in (torch.bfloat16, torch.float32):
        c = torch.full((M, N), 7.0, dtype=c_dtype, device="cuda")
        assert o.gemm_skinny(a, w, c, o.EPILOGUE_STORE, splits)
        torch.testing.assert_close(c.float().cpu(), ref.float().to(c_dtype).float(), **tol(c_dtype, ref))
        c2 = torch.empty_like(c)
        assert o.gemm_skinny(a, w, c2, o.EPILOGUE_STORE, splits)
        assert torch.equal(c, c2)
    res0 = torch.randn(M, N, generator=g)
    res = res0.clone().cuda()
    assert o.gemm_skinny(a, w, res, o.EPILOGUE_RESIDUAL_ADD, splits)
    torch.testing.assert_close(res.cpu(), (res0.double() + ref).float(), **tol(torch.float32, ref))
    h = torch.empty(M, N // 2, dtype=torch.bfloat16, device="cuda")
    assert o.gemm_skinny(a, w, h, o.EPILOGUE_GATED_SILU, splits)
    gated = P.swiglu(ref[:, 0::2], ref[:, 1::2])
    torch.testing.assert_close(h.float().cpu(), gated.float().to(torch.bfloat16).float(), **tol(torch.bfloat16, gated))
    assert o.gemm_skinny_status() == 0
    assert not o.gemm_skinny(torch.zeros(129, K, dtype=torch.bfloat16, device="cuda"), w, torch.empty(129, N, device="cuda"))


def test_decode_attention_reports_the_ctas_an_sm_holds():
    """The spans of decode attention are planned for what the GPU holds at once: the occupancy of the kernel
    for the head size (more for small heads than for large ones), 4 per SM as a stand-in for sizes that kernel
    does not take."""
    o = ops()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    small, large = o.resident_ctas("cuda:0", 64, 4), o.resident_ctas("cuda:0", 128, 4)
    assert small % sms == 0 and large % sms == 0 and small >= large >= sms
    assert o.resident_ctas("cuda:0", 48, 4) == 4 * sms            # no kernel for heads of 48: the stand-in
    assert o.resident_ctas("cuda:0", 64, 16) >= sms               # groups of more than 8 heads: the full-tile variant


@pytest.mark.parametrize("H, KVH, D, window", [(4, 2, 32, 0), (32, 8, 64, 0), (3, 1, 96, 0), (16, 1, 128, 0),
                                               (8, 8, 64, 0), (24, 2, 32, 0), (8, 2, 64, 100), (4, 1, 128, 33)])
@pytest.mark.parametrize("n_splits", [1, 2, 3, 8, 16])
def test_attention_decode_against_plain(H, KVH, D, window, n_splits):
    kv_lens = [1, 31, 32, 33, 64, 65, 300, 517]
    k_pool, v_pool, table, dense = _paged_setup(torch.bfloat16, len(kv_lens), kv_lens, KVH, D, n_pages=40, seed=D + H)
    g = torch.Generator().manual_seed(2)
    B = len(kv_lens)
    q = (torch.randn(B, H, D, generator=g) * 2).to(torch.bfloat16)
    refs = []
    for s, n in enumerate(kv_lens):
        k, v = dense[s]
        lo = max(0, n - window) if window else 0
        qq = q[s].float().reshape(1, H, D).expand(n - lo, H, D).contiguous()
        refs.append(P.causal_attention(qq, k[lo:], v[lo:])[-1])
    ref = torch.stack(refs).reshape(B, H * D)
    qkv = torch.cat([q.reshape(B, H * D), torch.randn(B, 2 * KVH * D).to(torch.bfloat16)], dim=1).cuda().contiguous()
    out = torch.empty(B, H * D, dtype=torch.bfloat16, device="cuda")
    lens = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    ops().attention_decode(qkv, qkv.shape[1], out, lens, table, k_pool, v_pool, H, KVH, D, window, n_splits)
    # probabilities are rounded to bfloat16 before they meet the values: 2^-8 of the largest output
    torch.testing.assert_close(out.float().cpu(), ref, rtol=2.0 ** -7, atol=2.0 ** -8 * float(ref.abs().max()))


@pytest.mark.parametrize("H, KVH, D, window", [(4, 2, 32, 0), (8, 2, 64, 0), (3, 1, 96, 0), (4, 4, 128, 0),
                                               (4, 1, 64, 37), (2, 1, 128, 200), (6, 2, 32, 64)])
def test_attention_prefill_against_plain(H, KVH, D, window):
    """Whole prompts, chunks that continue a cached prefix and single tokens in one packed batch."""
    kv_lens = [1, 64, 65, 300, 129, 517, 40]
    q_starts = [0, 0, 64, 101, 100, 0, 39]
    k_pool, v_pool, table, dense = _paged_setup(torch.bfloat16, len(kv_lens), kv_lens, KVH, D, n_pages=60, seed=D + H)
    g = torch.Generator().manual_seed(1)
    qs, refs, cu = [], [], [0]
    for s, (n, q0) in enumerate(zip(kv_lens, q_starts)):
        k, v = dense[s]
        q_full = (torch.randn(n, H, D, generator=g) * 2).to(torch.bfloat16).float()
        refs.append(P.causal_attention(q_full, k, v, window or None)[q0:])
        qs.append(q_full[q0:])
        cu.append(cu[-1] + n - q0)
    q = torch.cat(qs).reshape(-1, H * D)
    qkv = torch.cat([q, torch.randn(q.shape[0], 2 * KVH * D)], dim=1).to(torch.bfloat16).cuda().contiguous()
    out = torch.full((q.shape[0], H * D), 9.0, dtype=torch.bfloat16, device="cuda")
    ops().attention_prefill(qkv, qkv.shape[1], out, torch.tensor(cu, dtype=torch.int32, device="cuda"),
                            torch.tensor(kv_lens, dtype=torch.int32, device="cuda"), table, k_pool, v_pool,
                            len(kv_lens), max(n - q0 for n, q0 in zip(kv_lens, q_starts)), H, KVH, D, window)
    ref = torch.cat(refs).reshape(-1, H * D)
    torch.testing.assert_close(out.float().cpu(), ref, rtol=2.0 ** -7, atol=2.0 ** -8 * float(ref.abs().max()))


@pytest.mark.parametrize("H, KVH, D, pairing, window", [(8, 2, 64, "half", 0), (32, 8, 64, "half", 0), (4, 1, 128, "half", 70),
                                                        (6, 3, 32, "interleaved", 0), (3, 1, 96, "interleaved", 0),
                                                        (16, 1, 128, "interleaved", 0)])
@pytest.mark.parametrize("n_splits", [1, 4, 16])
def test_attention_decode_with_fused_rotation_and_cache_write(H, KVH, D, pairing, window, n_splits):
    """One kernel that rotates the step's queries, stores its key and value and attends must give what
    the rotation kernel followed by the attention kernel give: the same cache, the same output."""
    from gpullama3.java_b200.parts.position import PAIRING_CODES
    o = ops()
    kv_lens = [1, 2, 33, 64, 65, 300, 517]   # lengths after the step: the new token sits at kv_len - 1
    B = len(kv_lens)
    k_pool, v_pool, table, _ = _paged_setup(torch.bfloat16, B, kv_lens, KVH, D, n_pages=40, seed=D + H)
    g = torch.Generator().manual_seed(3)
    qkv = (torch.randn(B, (H + 2 * KVH) * D, generator=g) * 2).to(torch.bfloat16).cuda()
    inv = P.rope_inverse_frequencies(D, 5e5, None).to(torch.float32).cuda()
    lens = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    pos = lens - 1
    seq = torch.arange(B, dtype=torch.int32, device="cuda")
    code = PAIRING_CODES[pairing]
    assert o.attention_decode_rope_supported(torch.bfloat16, H, KVH, D, D, code)
    # two steps, reference: separate kernels
    k_ref, v_ref, q_ref = k_pool.clone(), v_pool.clone(), qkv.clone()
    o.rope_cache_write(q_ref, pos, seq, table, inv, k_ref, v_ref, H, KVH, D, D, code)
    want = torch.empty(B, H * D, dtype=torch.bfloat16, device="cuda")
    o.attention_decode(q_ref, q_ref.shape[1], want, lens, table, k_ref, v_ref, H, KVH, D, window, n_splits)
    # fused
    k_new, v_new, raw = k_pool.clone(), v_pool.clone(), qkv.clone()
    got = torch.empty_like(want)
    o.attention_decode_rope(raw, got, lens, table, k_new, v_new, inv, H, KVH, D, code, window, n_splits)
    assert torch.equal(raw, qkv)                         # the projections are left as they were
    assert torch.equal(k_new, k_ref) and torch.equal(v_new, v_ref)
    scale = float(want.float().abs().max())
    torch.testing.assert_close(got.float(), want.float(), rtol=2.0 ** -7, atol=2.0 ** -8 * scale)
    # a layer that reads another layer's cache: nothing is stored, the cached last position is attended
    got2 = torch.empty_like(want)
    k2, v2 = k_ref.clone(), v_ref.clone()
    o.attention_decode_rope(raw, got2, lens, table, k2, v2, inv, H, KVH, D, code, window, n_splits, write_cache=False)
    assert torch.equal(k2, k_ref) and torch.equal(v2, v_ref)
    torch.testing.assert_close(got2.float(), want.float(), rtol=2.0 ** -7, atol=2.0 ** -8 * scale)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("H, KVH, window", [(8, 2, 0), (4, 4, 0), (3, 1, 0), (4, 1, 37), (2, 1, 200), (2, 2, 129)])
def test_attention_prefill_on_tcgen05_against_plain(H, KVH, window, D):
    """The tensor-memory flash kernel (head sizes 64 and 128): whole prompts across several 128-row tiles and
    128-key blocks, chunks that continue a cached prefix, single tokens, windows; every wait inside must complete."""
    kv_lens = [1, 64, 65, 300, 129, 517, 40, 128, 700]
    q_starts = [0, 0, 64, 101, 100, 0, 39, 0, 256]
    k_pool, v_pool, table, dense = _paged_setup(torch.bfloat16, len(kv_lens), kv_lens, KVH, D, n_pages=60, seed=H + KVH)
    g = torch.Generator().manual_seed(1)
    qs, refs, cu = [], [], [0]
    for s, (n, q0) in enumerate(zip(kv_lens, q_starts)):
        k, v = dense[s]
        q_full = (torch.randn(n, H, D, generator=g) * 2).to(torch.bfloat16).float()
        refs.append(P.causal_attention(q_full, k, v, window or None)[q0:])
        qs.append(q_full[q0:])
        cu.append(cu[-1] + n - q0)
    q = torch.cat(qs).reshape(-1, H * D)
    qkv = torch.cat([q, torch.randn(q.shape[0], 2 * KVH * D)], dim=1).to(torch.bfloat16).cuda().contiguous()
    out = torch.full((q.shape[0], H * D), 9.0, dtype=torch.bfloat16, device="cuda")
    assert ops().attention_prefill_tc(qkv, qkv.shape[1], out, torch.tensor(cu, dtype=torch.int32, device="cuda"),
                                      torch.tensor(kv_lens, dtype=torch.int32, device="cuda"), table, k_pool, v_pool,
                                      len(kv_lens), max(n - q0 for n, q0 in zip(kv_lens, q_starts)), H, KVH, D, window)
    assert ops().attention_prefill_tc_status() == 0
    ref = torch.cat(refs).reshape(-1, H * D)
    torch.testing.assert_close(out.float().cpu(), ref, rtol=2.0 ** -7, atol=2.0 ** -8 * float(ref.abs().max()))


@pytest.mark.parametrize("D", [64, 128])
def test_attention_prefill_pairs_of_tiles_against_plain(D):
    """With enough work the tensor-memory kernel takes query tiles in pairs, one CTA per SM walking through many
    (pair, head, sequence) units: long and short sequences, a tile pair whose second tile is empty or partial,
    prefixes that are no multiple of the block, more units than SMs so that every CTA handles several."""
    H, KVH = 16, 4
    kv_lens = [1500, 129, 128, 257, 700, 64, 1, 385]
    q_starts = [0, 0, 0, 1, 300, 63, 0, 130]
    k_pool, v_pool, table, dense = _paged_setup(torch.bfloat16, len(kv_lens), kv_lens, KVH, D, n_pages=70, seed=11)
    g = torch.Generator().manual_seed(5)
    qs, refs, cu = [], [], [0]
    for s, (n, q0) in enumerate(zip(kv_lens, q_starts)):
        k, v = dense[s]
        q_full = (torch.randn(n, H, D, generator=g) * 2).to(torch.bfloat16).float()
        refs.append(P.causal_attention(q_full, k, v, None)[q0:])
        qs.append(q_full[q0:])
        cu.append(cu[-1] + n - q0)
    q = torch.cat(qs).reshape(-1, H * D)
    qkv = torch.cat([q, torch.randn(q.shape[0], 2 * KVH * D)], dim=1).to(torch.bfloat16).cuda().contiguous()
    out = torch.full((q.shape[0], H * D), 9.0, dtype=torch.bfloat16, device="cuda")
    max_q = max(n - q0 for n, q0 in zip(kv_lens, q_starts))
    assert -(-max_q // 256) * H * len(kv_lens) >= 148 * 4
    for _ in range(2):  # the second launch starts from the work counter the first one left
        assert ops().attention_prefill_tc(qkv, qkv.shape[1], out, torch.tensor(cu, dtype=torch.int32, device="cuda"),
                                          torch.tensor(kv_lens, dtype=torch.int32, device="cuda"), table, k_pool, v_pool,
                                          len(kv_lens), max_q, H, KVH, D, 0)
    assert ops().attention_prefill_tc_status() == 0
    ref = torch.cat(refs).reshape(-1, H * D)
    torch.testing.assert_close(out.float().cpu(), ref, rtol=2.0 ** -7, atol=2.0 ** -8 * float(ref.abs().max()))


def test_attention_decode_ignores_what_lies_beyond_a_sequence():
    """Slots are used again without clearing: stale or non-finite numbers after a sequence's last
    position (same page) and in pages of other sequences must not reach the output."""
    H, KVH, D = 8, 2, 64
    kv_lens = [37, 70]
    k_pool, v_pool, table, dense = _paged_setup(torch.bfloat16, 2, kv_lens, KVH, D, n_pages=8, seed=4)
    q = torch.randn(2, H * D).to(torch.bfloat16)
    qkv = torch.cat([q, torch.zeros(2, 2 * KVH * D, dtype=torch.bfloat16)], dim=1).cuda()
    lens = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    clean = torch.empty(2, H * D, dtype=torch.bfloat16, device="cuda")
    ops().attention_decode(qkv, qkv.shape[1], clean, lens, table, k_pool, v_pool, H, KVH, D, 0, 2)
    for s, n in enumerate(kv_lens):
        page = int(table[s, (n - 1) // 64])
        k_pool[page, :, n % 64:] = float("nan")
        v_pool[page, :, :, n % 64:] = float("inf")
    dirty = torch.empty_like(clean)
    ops().attention_decode(qkv, qkv.shape[1], dirty, lens, table, k_pool, v_pool, H, KVH, D, 0, 2)
    assert torch.equal(clean, dirty)


@pytest.mark.parametrize("V", [5, 384, 1000, 128256])
def test_argmax_first_maximum_wins(V):
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(6, V, generator=g)
    logits[1, V // 2] = logits[1, V - 1] = 9.0       # a tie: the lower index wins
    logits[2, 0] = 50.0
    logits[3, V - 1] = 50.0
    logits[4] = -float("inf")
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops().argmax_rows(logits.cuda(), out)
    assert out.tolist() == [P.argmax_first(r) if torch.isfinite(r).any() else 0 for r in logits]
    assert out.tolist()[1] == V // 2


@pytest.mark.parametrize("V, temperature", [(11, 1.0), (384, 0.8), (5003, 0.3)])
def test_temperature_sampling_is_the_inverse_cdf_in_index_order(V, temperature):
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(1, V, generator=g) * 2
    us = [0.0, 0.001, 0.25, 0.5, 0.75, 0.999, 0.99999994]
    rows = logits.repeat(len(us), 1).cuda()
    out = torch.empty(len(us), dtype=torch.int32, device="cuda")
    ops().sample_rows(rows, torch.tensor(us, dtype=torch.float32, device="cuda"), out, temperature, 1.0)
    p = P.temperature_softmax(logits[0], temperature).double()
    cdf = torch.cumsum(p, 0)
    for u, tok in zip(us, out.tolist()):
        want = P.sample_categorical(p.float(), u)
        lo = float(cdf[tok - 1]) if tok > 0 else 0.0
        # the same token, or a neighbour when u falls within rounding of a boundary of the cdf
        assert tok == want or min(abs(u - lo), abs(u - float(cdf[tok]))) < 1e-5, (u, tok, want)


@pytest.mark.parametrize("V, top_p, temperature, spread", [
    (9, 0.6, 1.0, 3.0), (384, 0.95, 0.8, 3.0), (5003, 0.9, 0.5, 3.0), (700, 0.05, 1.0, 3.0),
    (20011, 0.9, 1.0, 0.5),      # flat: every token passes the cutoff, the row itself is walked
    (128256, 0.95, 0.1, 2.0),    # peaked, the reference's default settings: a short list of candidates is gathered
    (40000, 0.99, 1.0, 1.5)])    # in between: thousands of candidates
def test_nucleus_sampling_matches_plain(V, top_p, temperature, spread):
    g = torch.Generator().manual_seed(V + 1)
    logits = torch.randn(1, V, generator=g) * spread
    logits[0, 5] = logits[0, 3]                      # equal probabilities are ordered by index
    us = [0.0, 0.1, 0.33, 0.5, 0.8, 0.95, 0.9999]
    rows = logits.repeat(len(us), 1).cuda()
    out = torch.empty(len(us), dtype=torch.int32, device="cuda")
    ops().sample_rows(rows, torch.tensor(us, dtype=torch.float32, device="cuda"), out, temperature, top_p)
    p = P.temperature_softmax(logits[0], temperature)
    n_candidates = int((p >= (1.0 - top_p) / (V - 1)).sum())
    assert {20011: n_candidates > 4093, 128256: n_candidates < 200, 40000: n_candidates > 1000}.get(V, True), n_candidates
    pl = p.tolist()
    order = sorted(range(V), key=lambda i: (-pl[i], i))
    csum = torch.cumsum(p[order].double(), 0)
    for u, tok in zip(us, out.tolist()):
        want = P.sample_top_p(p, top_p, u)
        if tok != want:   # allowed only when r falls within rounding of a boundary between neighbours
            kept = int((csum <= top_p).sum()) + 1
            r = u * float(csum[kept - 1])
            j = order.index(tok)
            assert j < kept and min(abs(r - float(csum[j])), abs(r - (float(csum[j - 1]) if j else 0.0))) < 1e-5, (u, tok, want)


def test_kernels_refuse_what_they_cannot_do():
    o = ops()
    from gpullama3.java_b200.kernels.ops import KernelError
    q = torch.zeros(1, 3 * 24, device="cuda")
    out = torch.zeros(1, 24, device="cuda")
    pool = torch.zeros(1, 1, 64, 24, device="cuda")
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(KernelError, match="unsupported size"):
        o.attention_paged(q, 72, out, z, z, z.reshape(1, 1), pool, pool.transpose(2, 3).contiguous(), 1, 1, 24, 0)   # head size not a step of 16
    # decode attention reads queries, keys and values 16 bytes at a time: a pointer off that grid is refused
    qb = torch.zeros(2, 3 * 64 + 8, dtype=torch.bfloat16, device="cuda")
    ob = torch.zeros(2, 64, dtype=torch.bfloat16, device="cuda")
    kb = torch.zeros(1, 1, 64, 64, dtype=torch.bfloat16, device="cuda")
    one = torch.ones(2, dtype=torch.int32, device="cuda")
    tab = torch.zeros(2, 1, dtype=torch.int32, device="cuda")
    o.attention_decode(qb, qb.shape[1], ob, one, tab, kb, kb.transpose(2, 3).contiguous(), 1, 1, 64, 0, 1)   # aligned: runs
    with pytest.raises(KernelError, match="unsupported size"):
        o.attention_decode(qb[:, 1:], qb.shape[1], ob, one, tab, kb, kb.transpose(2, 3).contiguous(), 1, 1, 64, 0, 1)
    with pytest.raises(KernelError):
        o.embed_gather(torch.zeros(4, 4), torch.zeros(1, dtype=torch.int32), torch.zeros(1, 4))   # CPU tensors
    with pytest.raises(KernelError, match="bad argument"):
        o.sample_rows(torch.zeros(1, 8, device="cuda"), torch.zeros(1, device="cuda"),
                      torch.zeros(1, dtype=torch.int32, device="cuda"), 0.0, 1.0)       # temperature 0 is argmax's job
