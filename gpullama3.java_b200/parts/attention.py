"""Grouped-query causal attention over the paged cache: the mixer of the Llama 3 decoder.

One run: project the normalised input to queries, keys and values with one fused weight
(inference/InferenceCore.java:78-80 of the reference project computes the three separately),
rotate queries and keys and store keys and values at each token's position (:83-101), attend over
everything the sequence has cached up to each token (:106-145), project back and add to the
residual stream (:148-151).  Sizes, the position encoding and an optional window are parameters."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import KVCacheNeed, KVView
from ..config.base import ConfigError
from ..kernels import fast, ops
from ..weights.loader import ParamSpec
from .base import Mixer, PositionEncoding, StepContext, register_mixer
from .linear import Linear


class GroupedQueryAttention(Mixer):
    graph_safe = True
    pad_safe = True

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, position: PositionEncoding,
                 window: int | None = None):
        if n_heads % n_kv_heads:
            raise ConfigError(f"n_heads {n_heads} must be a multiple of n_kv_heads {n_kv_heads}")
        # what no kernel takes is refused here, when the model is built, not at the first step
        if head_dim % ops.HEAD_DIM_STEP or not (0 < head_dim <= ops.MAX_HEAD_DIM):
            raise ConfigError(f"head_dim {head_dim}: the attention kernels take head sizes in steps of "
                              f"{ops.HEAD_DIM_STEP} up to {ops.MAX_HEAD_DIM}")
        if position.rotary_dim > min(head_dim, ops.MAX_ROTARY_DIM) or position.rotary_dim % 2:
            raise ConfigError(f"rotary_dim {position.rotary_dim} must be even and at most "
                              f"{min(head_dim, ops.MAX_ROTARY_DIM)} (head_dim {head_dim})")
        if window is not None and window < 1:
            raise ConfigError(f"window {window} must be at least 1 (or None for no window)")
        self.hidden_size, self.n_heads, self.n_kv_heads, self.head_dim = hidden_size, n_heads, n_kv_heads, head_dim
        self.position, self.window = position, window
        self.q_dim, self.kv_dim = n_heads * head_dim, n_kv_heads * head_dim
        self.qkv: Linear | None = None
        self.o: Linear | None = None

    def parameters(self):
        return {"q": ParamSpec((self.q_dim, self.hidden_size)), "k": ParamSpec((self.kv_dim, self.hidden_size)),
                "v": ParamSpec((self.kv_dim, self.hidden_size)), "o": ParamSpec((self.hidden_size, self.q_dim))}

    def children(self):
        return {"position": self.position}

    def cache_need(self):
        return KVCacheNeed(self.n_kv_heads, self.head_dim, self.window)

    def plan_decode(self, ctx: StepContext, cache: KVView) -> tuple[int, bool]:
        """How a decode step's attention is launched: into how many spans each sequence's keys are cut, and
        whether the kernel may be scheduled while its predecessor still runs.  Both follow from the number of
        sequences, this mixer's own kv heads and the longest sequence the step must be right for (its cache
        group's ``kv_capacity``: a recorded step is replayed until its page tables are outgrown)."""
        capacity = ctx.capacity(cache.group)
        if self.window:
            capacity = min(capacity, self.window)
        resident = ops.resident_ctas(ctx.device, self.head_dim, self.n_heads // self.n_kv_heads)
        splits = ops.attention_decode_splits(ctx.n_seqs, self.n_kv_heads, capacity, resident)
        return splits, ops.attention_decode_early_start(ctx.n_seqs, self.n_kv_heads, capacity, splits)

    def load(self, tensors, dtype, device):
        q, k, v, o = (tensors[n].to(device) for n in ("q", "k", "v", "o"))
        common = torch.float32 if (dtype == torch.float32 or torch.float32 in (q.dtype, k.dtype, v.dtype)) else q.dtype
        self.qkv = Linear(torch.cat([q.to(common), k.to(common), v.to(common)], dim=0).contiguous())
        self.o = Linear(o.to(torch.float32 if dtype == torch.float32 else o.dtype).contiguous())

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        return ctx.all_decode and self.qkv.links_with(ctx.n_tokens, ctx.dtype)

    def forward(self, x, ctx: StepContext, cache: KVView, residual, writes_cache=True, then_norm=None):
        table = ctx.page_tables[cache.group]
        out = ctx.empty((x.shape[0], self.q_dim), ctx.dtype)
        attended = False
        if isinstance(x, torch.Tensor) and not ctx.all_decode:
            # a prompt pass: projection, rotation and cache write as one product where its epilogue can do all three
            qkv = ctx.empty((x.shape[0], self.qkv.out_features), ctx.dtype)
            if not fast.try_projection_with_rope(x, self.qkv.weight, qkv, ctx, table, cache, self, writes_cache):
                self.qkv.into(x, qkv)
                ops.rope_cache_write(qkv, ctx.positions, ctx.seq_ids, table, self.position.inverse_frequencies(x.device),
                                     cache.k, cache.v, self.n_heads, self.n_kv_heads, self.head_dim,
                                     self.position.rotary_dim, self.position.pairing, write_cache=writes_cache)
        else:
            qkv = self.qkv.store(x, ctx.dtype, ctx.empty)  # [T, q_dim + 2 kv_dim]; queries are rotated in place below
            # a decode step: one kernel rotates, writes the cache and attends, where the sizes allow
            attended = fast.try_decode_attention_with_rope(qkv, out, ctx, table, cache, self, writes_cache)
            if not attended:
                ops.rope_cache_write(qkv, ctx.positions, ctx.seq_ids, table, self.position.inverse_frequencies(x.device),
                                     cache.k, cache.v, self.n_heads, self.n_kv_heads, self.head_dim,
                                     self.position.rotary_dim, self.position.pairing, write_cache=writes_cache)
        if not attended and not fast.try_attention(qkv, out, ctx, table, cache, self):
            # (the plain kernel: a step of few tokens cuts their keys into spans so that the GPU has CTAs to run)
            rows = x.shape[0] * self.n_heads
            splits = 1 if rows >= 1024 else max(1, min(16, 1024 // rows, ctx.capacity(cache.group) // 512))
            ops.attention_paged(qkv, qkv.shape[1], out, ctx.positions, ctx.seq_ids, table, cache.k, cache.v,
                                self.n_heads, self.n_kv_heads, self.head_dim, self.window or 0, n_splits=splits)
        return self.o.add_to(out, residual, then_norm)


register_mixer("attention", GroupedQueryAttention)
