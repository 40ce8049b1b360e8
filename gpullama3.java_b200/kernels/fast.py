"""Choice of the tensor-core kernels of the bfloat16 run.

``try_gemm`` and ``try_attention`` run the specialised sm_100a kernel that fits the operands and
return True, or return False when no specialised kernel takes these storage types or sizes (the
caller then runs the plain kernel, which takes every size).  The true 32-bit run never comes
here with anything but float32 operands and therefore always takes the plain kernels."""
from __future__ import annotations

import torch

from . import ops


def try_gemm(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epilogue: int) -> bool:
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    M = a.shape[0]
    if M <= 16:
        return ops.gemm_decode(a, w, c, epilogue)
    if M <= 128 and ops.gemm_skinny(a, w, c, epilogue):
        return True
    if M <= 64 and ops.gemm_decode(a, w, c, epilogue):
        return True
    return ops.gemm_tcgen05(a, w, c, epilogue)


def try_projection_with_rope(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, ctx, page_table, cache, mixer,
                             writes_cache: bool) -> bool:
    """A prompt pass's query/key/value projection with rotation and cache write in the product's epilogue, where the
    sizes allow (whole heads of 64 or 128 in 256-column tiles, a position encoding that offers its angles per pass)."""
    pos = mixer.position
    if (ctx.all_decode or x.dtype != torch.bfloat16 or pos.rotary_dim != mixer.head_dim or mixer.head_dim not in (64, 128)
            or not hasattr(pos, "angles")):
        return False
    if ops.gemm_tcgen05_k_spans(x.shape[0], w.shape[0], x.shape[1]) != 1:
        return False
    return ops.gemm_tcgen05_qkv_rope(x, w, qkv, ctx.positions, ctx.seq_ids, page_table, pos.angles(ctx),
                                     cache.k if writes_cache else None, cache.v if writes_cache else None,
                                     mixer.n_heads, mixer.n_kv_heads, mixer.head_dim, pos.pairing, writes_cache)


def try_decode_attention_with_rope(qkv, out, ctx, page_table, cache, mixer, writes_cache: bool) -> bool:
    """A decode step's rotation, cache write and attention in one kernel, where the sizes allow."""
    pos = mixer.position
    if not (ctx.all_decode and ops.attention_decode_rope_supported(qkv.dtype, mixer.n_heads, mixer.n_kv_heads,
                                                                   mixer.head_dim, pos.rotary_dim, pos.pairing)):
        return False
    splits, early = mixer.plan_decode(ctx, cache)
    ops.attention_decode_rope(qkv, out, ctx.kv_lens, page_table, cache.k, cache.v, pos.inverse_frequencies(qkv.device),
                              mixer.n_heads, mixer.n_kv_heads, mixer.head_dim, pos.pairing, mixer.window or 0, splits,
                              write_cache=writes_cache, early_start=early)
    return True


def try_attention(qkv, out, ctx, page_table, cache, mixer) -> bool:
    if ctx.all_decode and ops.attention_decode_supported(qkv.dtype, mixer.n_heads, mixer.n_kv_heads, mixer.head_dim):
        splits, early = mixer.plan_decode(ctx, cache)
        ops.attention_decode(qkv, qkv.shape[1], out, ctx.kv_lens, page_table, cache.k, cache.v, mixer.n_heads,
                             mixer.n_kv_heads, mixer.head_dim, mixer.window or 0, splits, early_start=early)
        return True
    if qkv.dtype == torch.bfloat16 and ops.attention_prefill_tc(
            qkv, qkv.shape[1], out, ctx.cu_seqlens, ctx.kv_lens, page_table, cache.k, cache.v, ctx.n_seqs,
            ctx.max_q_len, mixer.n_heads, mixer.n_kv_heads, mixer.head_dim, mixer.window or 0):
        return True
    if qkv.dtype == torch.bfloat16 and mixer.head_dim in (32, 64, 96, 128):
        ops.attention_prefill(qkv, qkv.shape[1], out, ctx.cu_seqlens, ctx.kv_lens, page_table, cache.k, cache.v,
                              ctx.n_seqs, ctx.max_q_len, mixer.n_heads, mixer.n_kv_heads, mixer.head_dim,
                              mixer.window or 0)
        return True
    return False
