"""Python faces of the CUDA kernels: each function checks its tensors and calls one exported C
function on torch's current stream.  There is no other implementation behind these names: on a
machine without a GPU or without the compiled libraries they raise."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from .build import KernelBuildError, library

F32, BF16 = 0, 1
PAGE_TOKENS = 64  # must equal b200::kPageTokens
# what the plain kernels, which take every size the others refuse, are built for
HEAD_DIM_STEP, MAX_HEAD_DIM = 16, 256   # attention_generic.cu
MAX_ROTARY_DIM = 512                    # rope_cache.cu

_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


_ERRORS = {
    10001: "bad argument",
    10002: "unsupported size",
    10003: "scratch too small",
    10004: "the call needs more scratch than the built-in array of the no-allocation entry point holds",
}

_functions: dict[str, ctypes._CFuncPtr] = {}

# C signatures: library, then argument types (the trailing stream is added for all)
_SIGNATURES = {
    "b200_embed_gather": ("embedding", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int]),
    "b200_rmsnorm": ("norm", [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float]),
    "b200_rope_cache_write": ("rope_cache", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "b200_attention_paged": ("attention_generic", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                                   c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                                   c_void_p]),
    "b200_gemm_generic": ("gemm_generic", [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                                           c_int, c_int, c_int, c_int]),
    "b200_gemm_decode": ("gemm_decode", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                         c_int]),
    "b200_gemm_decode_linked": ("gemm_decode", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                c_int, c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_int, c_void_p,
                                                c_int, c_void_p]),
    "b200_gemm_tcgen05": ("gemm_tcgen05", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_int, c_int, c_int, c_int]),
    "b200_gemm_tcgen05_qkv_rope": ("gemm_tcgen05", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p,
                                                    c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                    c_int, c_int, c_int]),
    "b200_rope_angles": ("rope_cache", [c_void_p, c_void_p, c_void_p, c_int, c_int]),
    "b200_gemm_skinny": ("gemm_skinny_tcgen05", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                                 c_int, c_int, c_int]),
    "b200_attention_decode": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                   c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_int,
                                                   c_int, c_int, c_int]),
    "b200_attention_prefill": ("attention_prefill", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                     c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int]),
    "b200_attention_decode_rope": ("attention_decode", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                        c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_int,
                                                        c_int, c_int, c_int, c_void_p, c_int, c_int, c_int]),
    "b200_attention_prefill_tc": ("attention_prefill_tcgen05", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                                c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                                                c_int, c_int, c_int, c_int]),
    "b200_random_fill": ("random_init", [c_void_p, c_int, ctypes.c_longlong, ctypes.c_ulonglong, c_float, c_float]),
    "b200_argmax_rows": ("sampling", [c_void_p, c_int, c_void_p, c_int, c_int]),
    "b200_sample_rows": ("sampling", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p]),
}


def _fn(name: str):
    f = _functions.get(name)
    if f is None:
        lib_name, argtypes = _SIGNATURES[name]
        lib = library(lib_name)
        try:
            f = getattr(lib, name)
        except AttributeError as e:
            raise KernelBuildError(f"{name} is not exported by the {lib_name} kernel library") from e
        f.argtypes = list(argtypes) + [c_void_p]
        f.restype = c_int
        n_args = len(f.argtypes)

        def checked(*args, _f=f, _n=n_args, _name=name):
            if len(args) != _n:  # ctypes lets extra arguments through, which shifts the stream pointer
                raise TypeError(f"{_name} takes {_n} arguments, got {len(args)}")
            if _profile is None:
                return _f(*args)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            status = _f(*args)
            e1.record()
            _profile.append((_name, e0, e1))
            return status

        f = _functions[name] = checked
    return f


_profile: list | None = None   # (function, start event, end event) per launch while profiling is on


def profile_start() -> None:
    """From now on every launch issued through these functions is bracketed by CUDA events on its stream.  Launches
    replayed from a CUDA graph are not seen: profile with graphs off."""
    global _profile
    _profile = []


def profile_stop() -> dict[str, tuple[int, float]]:
    """Ends profiling; ``{function: (launches, total device ms)}``."""
    global _profile
    rows, _profile = _profile or [], None
    torch.cuda.synchronize()
    out: dict[str, tuple[int, float]] = {}
    for name, e0, e1 in rows:
        n, ms = out.get(name, (0, 0.0))
        out[name] = (n + 1, ms + e0.elapsed_time(e1))
    return out


_launches = 0
_launches_by_kernel: dict[str, int] = {}


def launch_count() -> int:
    """How many kernel launches this process has issued through these functions."""
    return _launches


def launches_by_kernel() -> dict[str, int]:
    """The same count per kernel function (a copy).  A launch recorded into a CUDA graph counts once, when it
    is recorded.  Decode attention that was told not to start early counts under ``<name>:late``."""
    return dict(_launches_by_kernel)


def _check(status: int, name: str) -> None:
    global _launches
    _launches += 1
    _launches_by_kernel[name] = _launches_by_kernel.get(name, 0) + 1
    if status != 0:
        what = _ERRORS.get(status)
        if what is None:
            what = f"CUDA error {status}"
        raise KernelError(f"{name}: {what}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream's handle.  Asked for at every launch (a graph capture changes it), so through the
    two plain C calls where this torch has them: building a ``torch.cuda.Stream`` object costs several microseconds,
    which a pass of a hundred short kernels feels."""
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels store float32 or bfloat16, not {dtype}") from None


def _dev(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors only; there is no CPU path")


# --------------------------------------------------------------------------- embedding, norm
def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = table[tokens[t]] into the float32 residual stream.  tokens int32 [T]."""
    _dev(table, tokens, out)
    assert out.dtype == torch.float32 and tokens.dtype == torch.int32
    assert table.is_contiguous() and out.is_contiguous()
    n, dim = out.shape
    _check(_fn("b200_embed_gather")(table.data_ptr(), dtype_code(table.dtype), tokens.data_ptr(), out.data_ptr(),
                                    n, dim, table.shape[0], _stream()), "embed_gather")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> None:
    """out[r] = weight * x[rows[r]] / sqrt(mean(x^2) + eps).  x float32 [T, dim]."""
    _dev(x, weight, out, rows)
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous() and weight.is_contiguous()
    n_rows, dim = out.shape
    assert x.shape[1] == dim and weight.numel() == dim
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.numel() == n_rows
    _check(_fn("b200_rmsnorm")(x.data_ptr(), weight.data_ptr(), dtype_code(weight.dtype), out.data_ptr(),
                               dtype_code(out.dtype), rows.data_ptr() if rows is not None else None, n_rows, dim,
                               float(eps), _stream()), "rmsnorm")


# --------------------------------------------------------------------------- position encoding + cache write
def rope_cache_write(qkv: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor, page_table: torch.Tensor,
                     inv_freq: torch.Tensor, k_pool: torch.Tensor | None, v_pool: torch.Tensor | None, n_heads: int,
                     n_kv_heads: int, head_dim: int, rotary_dim: int, pairing: int, write_cache: bool = True) -> None:
    """Rotate the queries of ``qkv`` [T, (H + 2 KVH) D] in place; write rotated keys and the values
    into the cache pages of their positions."""
    _dev(qkv, positions, seq_ids, page_table, inv_freq, k_pool, v_pool)
    assert qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() >= max(rotary_dim // 2, 0)
    assert page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.is_contiguous()
    if write_cache:
        assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype
        assert k_pool.is_contiguous() and v_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
        assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    _check(_fn("b200_rope_cache_write")(
        qkv.data_ptr(), dtype_code(qkv.dtype), positions.data_ptr(), seq_ids.data_ptr(), page_table.data_ptr(),
        page_table.shape[1], inv_freq.data_ptr(), k_pool.data_ptr() if write_cache else None,
        v_pool.data_ptr() if write_cache else None, qkv.shape[0], n_heads, n_kv_heads, head_dim, rotary_dim, pairing,
        1 if write_cache else 0, _stream()), "rope_cache_write")


# --------------------------------------------------------------------------- attention
def attention_paged(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, positions: torch.Tensor,
                    seq_ids: torch.Tensor, page_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                    n_heads: int, n_kv_heads: int, head_dim: int, window: int = 0, n_splits: int = 1) -> None:
    """Causal grouped-query attention of every token of ``q`` over the cached keys 0..position of
    its sequence.  q: rows of ``q_row_stride`` elements whose first H*D are the rotated queries.
    ``n_splits`` > 1 cuts every token's keys into that many spans, one CTA each, merged by a second kernel (a decode
    step: few tokens, long rows of keys)."""
    _dev(q, out, positions, seq_ids, page_table, k_pool, v_pool)
    assert out.is_contiguous() and out.shape[1] == n_heads * head_dim and out.dtype == q.dtype == k_pool.dtype
    assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
    assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    scratch = None
    if n_splits > 1:
        scratch = torch.empty(out.shape[0] * n_heads * n_splits * (head_dim + 2), dtype=torch.float32, device=q.device)
    _check(_fn("b200_attention_paged")(
        q.data_ptr(), q_row_stride, out.data_ptr(), dtype_code(q.dtype), positions.data_ptr(), seq_ids.data_ptr(),
        page_table.data_ptr(), page_table.shape[1], k_pool.data_ptr(), v_pool.data_ptr(), out.shape[0], n_heads,
        n_kv_heads, head_dim, int(window), int(n_splits), scratch.data_ptr() if scratch is not None else None, _stream()),
        "attention_paged")


# --------------------------------------------------------------------------- matrix products
EPILOGUE_STORE, EPILOGUE_RESIDUAL_ADD, EPILOGUE_GATED_SILU = 0, 1, 2


def gemm_generic(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE) -> None:
    """c = a @ w.T (store), c += a @ w.T (residual add, c float32) or c = silu(gate) * up with
    gate/up rows interleaved in w.  32-bit FMA accumulation, no tensor cores."""
    _dev(a, w, c)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1
    assert c.shape[0] == M and c.shape[1] == (N // 2 if epilogue == EPILOGUE_GATED_SILU else N)
    _check(_fn("b200_gemm_generic")(
        a.data_ptr(), dtype_code(a.dtype), a.stride(0), w.data_ptr(), dtype_code(w.dtype), w.stride(0), c.data_ptr(),
        dtype_code(c.dtype), c.stride(0), M, N, K, epilogue, _stream()), "gemm_generic")


def gemm_decode(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE) -> bool:
    """The decode-step matrix product (bfloat16 operands, at most 64 tokens, K a multiple of 32).
    Returns False, having done nothing, for operands it does not take."""
    M, K = a.shape
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or M > 64 or K % 32 or a.stride(1) != 1
            or w.stride(1) != 1 or a.stride(0) % 8 or w.stride(0) % 8 or (a.data_ptr() | w.data_ptr()) & 15):
        return False
    _dev(a, w, c)
    N = w.shape[0]
    assert w.shape[1] == K and c.stride(1) == 1 and c.shape[0] == M
    assert c.shape[1] == (N // 2 if epilogue == EPILOGUE_GATED_SILU else N)
    _check(_fn("b200_gemm_decode")(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(),
                                   dtype_code(c.dtype), c.stride(0), M, N, K, epilogue, _stream()), "gemm_decode")
    return True


def gemm_decode_links(n_rows: int, w: torch.Tensor) -> bool:
    """Whether ``gemm_decode_linked`` takes a product of ``n_rows`` bfloat16 rows with ``w``."""
    return (w.dtype == torch.bfloat16 and n_rows <= 16 and w.shape[1] % 32 == 0 and w.stride(1) == 1
            and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0)


def gemm_decode_partials(n_rows: int, n_out: int) -> int:
    """How many partial sums of squares per row the residual product [n_rows, n_out] leaves."""
    lib = library("gemm_decode")
    return int(lib.b200_gemm_decode_ctas(n_rows, n_out))


def gemm_decode_linked(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int, *, row_factors=None,
                       emit=None) -> None:
    """``gemm_decode`` as one half, or both, of an RMSNorm split between two products (at most 16 rows).

    ``row_factors = (partials [M, P] float32, eps, dim)``: the rows of ``a`` are x * w of a norm; every
    sum of row t is multiplied by rsqrt(sum(partials[t]) / dim + eps) before the epilogue.
    ``emit = (norm_weight [N], act [M, N] bfloat16, partials [M, gemm_decode_partials(M, N)] float32)``
    (residual epilogue only): after c += a w^T, act = bfloat16(c * norm_weight) and partials hold each
    CTA's sum of c^2 per row."""
    M, K = a.shape
    N = w.shape[0]
    _dev(a, w, c)
    assert a.dtype == torch.bfloat16 and gemm_decode_links(M, w) and a.stride(1) == 1 and a.stride(0) % 8 == 0
    assert w.shape[1] == K and c.stride(1) == 1 and c.shape[0] == M and a.data_ptr() % 16 == 0
    assert c.shape[1] == (N // 2 if epilogue == EPILOGUE_GATED_SILU else N)
    in_p, n_in, eps, dim = None, 0, 0.0, 0
    if row_factors is not None:
        part, eps, dim = row_factors
        assert part.dtype == torch.float32 and part.is_contiguous() and part.shape[0] == M
        in_p, n_in = part.data_ptr(), part.shape[1]
    out_w, out_w_dtype, out_act, ld_act, out_p = None, 0, None, 0, None
    if emit is not None:
        nw, act, part_out = emit
        assert epilogue == EPILOGUE_RESIDUAL_ADD and nw.numel() == N and nw.is_contiguous()
        assert act.dtype == torch.bfloat16 and act.shape == (M, N) and act.stride(1) == 1
        assert part_out.dtype == torch.float32 and part_out.is_contiguous()
        assert tuple(part_out.shape) == (M, gemm_decode_partials(M, N))
        out_w, out_w_dtype, out_act, ld_act, out_p = nw.data_ptr(), dtype_code(nw.dtype), act.data_ptr(), act.stride(0), part_out.data_ptr()
    _check(_fn("b200_gemm_decode_linked")(
        a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), dtype_code(c.dtype), c.stride(0), M, N, K,
        epilogue, in_p, n_in, float(eps), int(dim), out_w, out_w_dtype, out_act, ld_act, out_p, _stream()),
        "gemm_decode_linked")


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE,
                 tile_width: int = 0, k_spans: int = 0, cta_pair: int = 0) -> bool:
    """The prefill matrix product on tcgen05 tensor cores (bfloat16 operands, rows 16-byte aligned).
    ``tile_width``: 256, 128 or 64 output columns per tile; 0 lets the shape decide (narrower tiles when the
    widest would leave SMs without one).  ``k_spans``: 2 or 4 cuts K among the CTAs of a cluster, which add their
    partial tiles in a fixed order (few tiles, long K); 1 never; 0 lets the shape decide.  ``cta_pair``: 1 computes
    tiles of 256 rows by pairs of CTAs that each load half of the weight stage (tile_width 256 or 128); -1 never;
    0 lets the shape decide.
    Returns False, having done nothing, for operands it does not take."""
    M, K = a.shape
    lda, a_inner = a.stride()
    ldw, w_inner = w.stride()
    pa, pw = a.data_ptr(), w.data_ptr()
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or K % 8 or K < 8 or a_inner != 1 or w_inner != 1
            or lda % 8 or ldw % 8 or (pa | pw) & 15):
        return False
    if epilogue == EPILOGUE_GATED_SILU and c.dtype != torch.bfloat16:
        return False
    _dev(a, w, c)
    N, Kw = w.shape
    ldc, c_inner = c.stride()
    assert Kw == K and c_inner == 1 and c.shape == (M, N // 2 if epilogue == EPILOGUE_GATED_SILU else N)
    _check(_fn("b200_gemm_tcgen05")(pa, lda, pw, ldw, c.data_ptr(), dtype_code(c.dtype), ldc, M, N, K, epilogue,
                                    tile_width, k_spans, cta_pair, _stream()), "gemm_tcgen05")
    return True


def rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor, half: int) -> torch.Tensor:
    """float32 [half, T, 2]: cosine and sine of position * frequency for every pair of a head and every token of a
    pass, evaluated as the rotation kernels evaluate them (pair-major: the tokens of a warp read neighbours)."""
    _dev(positions, inv_freq)
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32 and inv_freq.numel() >= half > 0
    out = torch.empty((half, positions.numel(), 2), dtype=torch.float32, device=positions.device)
    _check(_fn("b200_rope_angles")(positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), positions.numel(), half, _stream()),
           "rope_angles")
    return out


_UNSUPPORTED = 10002   # kErrUnsupportedSize: the kernel leaves these operands to another one


def gemm_tcgen05_qkv_rope(a: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, positions: torch.Tensor,
                          seq_ids: torch.Tensor, page_table: torch.Tensor, angles: torch.Tensor,
                          k_pool: torch.Tensor | None, v_pool: torch.Tensor | None, n_heads: int, n_kv_heads: int,
                          head_dim: int, pairing: int, write_cache: bool = True) -> bool:
    """The query/key/value projection of a prompt pass on tcgen05 tensor cores with the rotation and the cache
    write in its epilogue: ``qkv`` [T, (H + 2 KVH) D] receives the rotated queries (its key and value columns stay
    unwritten), rotated keys and the values go to the cache pages of their positions.  ``angles``: ``rope_angles`` of
    the pass.  Returns False, having done nothing, for shapes it does not take (head sizes other than 64 and 128, a
    product of few tiles): the caller then runs the product and ``rope_cache_write``."""
    M, K = a.shape
    N = (n_heads + 2 * n_kv_heads) * head_dim
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16 or head_dim not in (64, 128)
            or K % 8 or K < 8 or a.stride(1) != 1 or w.stride(1) != 1 or a.stride(0) % 8 or w.stride(0) % 8
            or qkv.stride(0) % 8 or (a.data_ptr() | w.data_ptr() | qkv.data_ptr()) & 15):
        return False
    _dev(a, w, qkv, positions, seq_ids, page_table, angles, k_pool, v_pool)
    assert tuple(w.shape) == (N, K) and tuple(qkv.shape) == (M, N) and qkv.stride(1) == 1
    assert positions.dtype == seq_ids.dtype == page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.is_contiguous()
    assert positions.numel() == M and seq_ids.numel() == M
    assert angles.dtype == torch.float32 and angles.is_contiguous() and tuple(angles.shape) == (head_dim // 2, M, 2)
    if write_cache:
        assert k_pool.dtype == v_pool.dtype == torch.bfloat16 and k_pool.is_contiguous() and v_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
        assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    status = _fn("b200_gemm_tcgen05_qkv_rope")(
        a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), qkv.data_ptr(), qkv.stride(0), M, K, positions.data_ptr(),
        seq_ids.data_ptr(), page_table.data_ptr(), page_table.shape[1], angles.data_ptr(),
        k_pool.data_ptr() if write_cache else None, v_pool.data_ptr() if write_cache else None, n_heads, n_kv_heads,
        head_dim, pairing, 1 if write_cache else 0, _stream())
    if status == _UNSUPPORTED:
        return False
    _check(status, "gemm_tcgen05_qkv_rope")
    return True


def gemm_tcgen05_k_spans(M: int, N: int, K: int) -> int:
    """Into how many spans ``gemm_tcgen05`` cuts K for this shape when it is left the choice (1: it does not)."""
    return int(library("gemm_tcgen05").b200_gemm_tcgen05_k_spans(M, N, K))


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int = EPILOGUE_STORE,
                k_splits: int | None = None) -> bool:
    """The few-token matrix product on tcgen05 tensor cores (bfloat16 operands, at most 128 tokens,
    rows 16-byte aligned).  Returns False, having done nothing, for operands it does not take."""
    M, K = a.shape
    if (a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or M > 128 or K % 8 or K < 8 or a.stride(1) != 1
            or w.stride(1) != 1 or a.stride(0) % 8 or w.stride(0) % 8 or (a.data_ptr() | w.data_ptr()) & 15):
        return False
    if epilogue == EPILOGUE_GATED_SILU and c.dtype != torch.bfloat16:
        return False
    _dev(a, w, c)
    N = w.shape[0]
    assert w.shape[1] == K and c.stride(1) == 1 and c.shape[0] == M
    assert c.shape[1] == (N // 2 if epilogue == EPILOGUE_GATED_SILU else N)
    fn = _fn("b200_gemm_skinny")
    if k_splits is None:
        k_splits = library("gemm_skinny_tcgen05").b200_gemm_skinny_splits(M, N, K, _sm_count(a.device))
    _check(fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), c.data_ptr(), dtype_code(c.dtype), c.stride(0), M, N,
              K, epilogue, k_splits, _stream()), "gemm_skinny")
    return True


_sm_counts: dict = {}


def _sm_count(device) -> int:
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def gemm_skinny_status() -> int:
    lib = library("gemm_skinny_tcgen05")
    lib.b200_gemm_skinny_status.restype = c_int
    return int(lib.b200_gemm_skinny_status())


def gemm_tcgen05_status() -> int:
    """0 when every wait inside the tensor-core GEMM completed since the last call; synchronises."""
    lib = library("gemm_tcgen05")
    lib.b200_gemm_tcgen05_status.restype = c_int
    return int(lib.b200_gemm_tcgen05_status())


def attention_decode_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (32, 64, 96, 128) and n_heads // n_kv_heads <= 16


_ctas_per_sm: dict = {}


def resident_ctas(device, head_dim: int = 64, group: int = 4, fused: bool = True) -> int:
    """The number of CTAs of decode attention the GPU holds at once, which is what the spans are planned for: the
    occupancy the driver reports for the kernel of these sizes (heads of 64 hold four per SM, heads of 128 two)
    times the SMs.  Four per SM for sizes that kernel does not take."""
    key = (head_dim, group > 8, fused)
    per_sm = _ctas_per_sm.get(key)
    if per_sm is None:
        query = library("attention_decode").b200_attention_decode_ctas_per_sm
        query.argtypes, query.restype = [c_int, c_int, c_int], c_int
        per_sm = _ctas_per_sm[key] = query(head_dim, group, 1 if fused else 0) or 4
    return per_sm * _sm_count(torch.device(device))


def attention_decode_splits(n_seqs: int, n_kv_heads: int, max_kv_len: int, resident_ctas: int) -> int:
    """How many spans each sequence's keys are cut into.  The grid (spans x kv heads x sequences)
    should fill the GPU in one wave (``resident_ctas``) without spilling into a second one.  Up to 16 spans a
    span may be as short as two blocks of 32 keys (a short context at a small batch is otherwise a handful of CTAs
    walking their keys one block after the other: batch 1 at 1,024 keys 0.705 -> 0.677 ms per step with 8 spans
    instead of 4); beyond 16 a span keeps at least 8 blocks so that its start-up and the merge pay (batch 1 at
    4,096 keys: 16 spans 0.713 ms, 32 spans 0.717, 64 spans 0.771)."""
    blocks = max(1, (max_kv_len + 31) // 32)
    cap = max(1, resident_ctas // max(1, n_seqs * n_kv_heads))
    want = max(1, min(cap, 64, max(blocks // 8, min(16, blocks // 2))))
    p = 1
    while p * 2 <= want:
        p *= 2
    return p


def attention_decode_early_start(n_seqs: int, n_kv_heads: int, max_kv_len: int, n_splits: int) -> bool:
    """Whether the decode attention may be scheduled while the kernel before it still runs.  A grid
    that fills the GPU with long spans (48 blocks of 32 keys or more) should find it empty instead:
    started early, its CTAs settle unevenly among the predecessor's and the fullest SMs finish late
    (batch 64 at 4,096 keys: 203 against 142 us per layer)."""
    blocks_per_span = (max_kv_len + 31) // 32 // max(1, n_splits)
    return not (n_seqs * n_kv_heads * n_splits >= 256 and blocks_per_span >= 48)


def attention_decode_rope_supported(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                                    pairing: int) -> bool:
    """Whether the decode kernel can also do the step's rotation and cache write."""
    return (attention_decode_supported(dtype, n_heads, n_kv_heads, head_dim) and rotary_dim == head_dim
            and (pairing == 0 or head_dim in (64, 128)))


def attention_decode_rope(qkv: torch.Tensor, out: torch.Tensor, kv_lens: torch.Tensor, page_table: torch.Tensor,
                          k_pool: torch.Tensor, v_pool: torch.Tensor, inv_freq: torch.Tensor, n_heads: int,
                          n_kv_heads: int, head_dim: int, pairing: int, window: int, n_splits: int,
                          write_cache: bool = True, scratch: torch.Tensor | None = None,
                          early_start: bool = True) -> None:
    """Decode attention that rotates the step's queries itself and, with ``write_cache``, stores the
    step's rotated key and its value at position kv_lens[i] - 1 of sequence i.  ``qkv``: the raw
    projections [n_seqs, (n_heads + 2 n_kv_heads) head_dim] (left untouched)."""
    _dev(qkv, out, kv_lens, page_table, k_pool, v_pool, inv_freq)
    n_seqs = out.shape[0]
    assert qkv.dtype == out.dtype == k_pool.dtype == torch.bfloat16 and out.is_contiguous() and qkv.is_contiguous()
    assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim and inv_freq.dtype == torch.float32
    assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
    assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    need = n_seqs * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0
    if need and (scratch is None or scratch.numel() < need):
        scratch = torch.empty(need, dtype=torch.float32, device=qkv.device)
    _check(_fn("b200_attention_decode_rope")(
        qkv.data_ptr(), qkv.shape[1], out.data_ptr(), kv_lens.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        k_pool.data_ptr(), v_pool.data_ptr(), scratch.data_ptr() if need else None, scratch.numel() if need else 0,
        n_seqs, n_heads, n_kv_heads, head_dim, int(window), n_splits, inv_freq.data_ptr(), pairing,
        1 if write_cache else 0, 1 if early_start else 0, _stream()),
        "attention_decode_rope" if early_start else "attention_decode_rope:late")


def attention_decode(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, kv_lens: torch.Tensor,
                     page_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, n_heads: int,
                     n_kv_heads: int, head_dim: int, window: int, n_splits: int,
                     scratch: torch.Tensor | None = None, early_start: bool = True) -> None:
    """One query token per sequence (row i of q belongs to sequence i) over kv_lens[i] cached keys.
    ``scratch``: float32 workspace for the spans' partial results (allocated here when absent).
    ``early_start``: see ``attention_decode_early_start``."""
    _dev(q, out, kv_lens, page_table, k_pool, v_pool)
    n_seqs = out.shape[0]
    assert q.dtype == out.dtype == k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
    assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    need = n_seqs * n_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0
    if need and (scratch is None or scratch.numel() < need):
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    _check(_fn("b200_attention_decode")(
        q.data_ptr(), q_row_stride, out.data_ptr(), kv_lens.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        k_pool.data_ptr(), v_pool.data_ptr(), scratch.data_ptr() if need else None, scratch.numel() if need else 0,
        n_seqs, n_heads, n_kv_heads, head_dim, int(window), n_splits, 1 if early_start else 0, _stream()),
        "attention_decode" if early_start else "attention_decode:late")


def attention_prefill(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, cu_seqlens: torch.Tensor,
                      kv_lens: torch.Tensor, page_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                      n_seqs: int, max_q_len: int, n_heads: int, n_kv_heads: int, head_dim: int, window: int) -> None:
    """Causal attention of packed query tokens: sequence i owns rows cu_seqlens[i]..cu_seqlens[i+1],
    which are its last positions (kv_lens[i] - q_len .. kv_lens[i] - 1); keys come from the cache."""
    _dev(q, out, cu_seqlens, kv_lens, page_table, k_pool, v_pool)
    assert q.dtype == out.dtype == k_pool.dtype == torch.bfloat16 and out.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
    assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    _check(_fn("b200_attention_prefill")(
        q.data_ptr(), q_row_stride, out.data_ptr(), cu_seqlens.data_ptr(), kv_lens.data_ptr(), page_table.data_ptr(),
        page_table.shape[1], k_pool.data_ptr(), v_pool.data_ptr(), n_seqs, max_q_len, n_heads, n_kv_heads, head_dim,
        int(window), _stream()), "attention_prefill")


def attention_prefill_tc(q: torch.Tensor, q_row_stride: int, out: torch.Tensor, cu_seqlens: torch.Tensor,
                         kv_lens: torch.Tensor, page_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                         n_seqs: int, max_q_len: int, n_heads: int, n_kv_heads: int, head_dim: int, window: int) -> bool:
    """``attention_prefill`` on tcgen05 tensor cores (head_dim 64 or 128).  Returns False, having done
    nothing, for sizes it does not take."""
    if head_dim not in (64, 128) or q.dtype != torch.bfloat16 or q_row_stride % 8 or (q.data_ptr() | out.data_ptr()) & 15:
        return False
    _dev(q, out, cu_seqlens, kv_lens, page_table, k_pool, v_pool)
    assert out.dtype == k_pool.dtype == torch.bfloat16 and out.is_contiguous() and k_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (n_kv_heads, PAGE_TOKENS, head_dim)
    assert tuple(v_pool.shape[1:]) == (n_kv_heads, head_dim, PAGE_TOKENS)
    _check(_fn("b200_attention_prefill_tc")(
        q.data_ptr(), q_row_stride, out.shape[0], out.data_ptr(), cu_seqlens.data_ptr(), kv_lens.data_ptr(),
        page_table.data_ptr(), page_table.shape[1], k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0], n_seqs,
        max_q_len, n_heads, n_kv_heads, head_dim, int(window), _stream()), "attention_prefill_tc")
    return True


def attention_prefill_tc_status() -> int:
    lib = library("attention_prefill_tcgen05")
    lib.b200_attention_prefill_tc_status.restype = c_int
    return int(lib.b200_attention_prefill_tc_status())


# --------------------------------------------------------------------------- random weights
def random_fill(out: torch.Tensor, key: int, scale: float, offset: float) -> None:
    """out.flat[i] = offset + scale * (sum of sixteen 16-bit fields of the splitmix64 sequence of ``key`` at 4i..4i+3,
    centred): the numbers ``weights.random_init.random_values`` makes on the CPU, bit for bit."""
    _dev(out)
    assert out.is_contiguous()
    _check(_fn("b200_random_fill")(out.data_ptr(), dtype_code(out.dtype), out.numel(), key & ((1 << 64) - 1),
                                   float(scale), float(offset), _stream()), "random_fill")


# --------------------------------------------------------------------------- sampling
def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of logits[r] (float32 [R, V]); out int32 [R]."""
    _dev(logits, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    _check(_fn("b200_argmax_rows")(logits.data_ptr(), logits.stride(0), out.data_ptr(), logits.shape[0],
                                   logits.shape[1], _stream()), "argmax_rows")


def sample_rows(logits: torch.Tensor, uniforms: torch.Tensor, out: torch.Tensor, temperature: float,
                top_p: float) -> None:
    """Temperature softmax and inverse-CDF draw (nucleus when 0 < top_p < 1) per row."""
    _dev(logits, uniforms, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert uniforms.dtype == torch.float32 and uniforms.numel() == logits.shape[0]
    scratch = None
    if 0.0 < top_p < 1.0:  # nucleus: the row's probabilities are kept in workspace between the passes
        scratch = torch.empty(logits.shape[0] * logits.shape[1], dtype=torch.float32, device=logits.device)
    _check(_fn("b200_sample_rows")(logits.data_ptr(), logits.stride(0), uniforms.data_ptr(), out.data_ptr(),
                                   logits.shape[0], logits.shape[1], float(temperature), float(top_p),
                                   scratch.data_ptr() if scratch is not None else None, _stream()),
           "sample_rows")
