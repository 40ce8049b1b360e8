"""The step function: a batch of sequences, each bringing its next tokens, run as one packed
batch from the cache; logits come back for the places that were asked for.

The same function serves whole prompts of unequal length, chunks that continue a cached prefix
and single decoded tokens: each token carries its own position and sequence, so nothing depends
on how tokens were cut into steps or on what else is in the batch.  The reference's step is one
token of one sequence (``forward(state, token, position)``, model/Model.java:61 of the reference
project) and feeds prompts through it token by token (inference/InferenceEngine.java:309-322)."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.pages import PAGE_TOKENS
from ..cache.sequence_cache import SequenceCache
from ..parts.base import StepContext


class StepError(ValueError):
    """The step was refused before anything ran (bad tokens, bad places, unknown slot)."""


@dataclass
class SequenceInput:
    slot: int
    tokens: list[int]
    want: list[int] = field(default_factory=list)  # places among ``tokens`` whose logits are wanted


def build_context(dtype, device, cache: SequenceCache, slots: list[int], start_pos: list[int],
                  token_lists: list, logit_rows: list[int]) -> tuple[StepContext, torch.Tensor | None]:
    """Pack one pass into a StepContext.  All integers go to the device in one copy."""
    n = len(slots)
    q_lens = [len(t) for t in token_lists]
    T = sum(q_lens)
    tokens = np.concatenate([np.asarray(t, dtype=np.int32) for t in token_lists])
    positions = np.concatenate([np.arange(s, s + q, dtype=np.int32) for s, q in zip(start_pos, q_lens)])
    seq_ids = np.repeat(np.arange(n, dtype=np.int32), q_lens)
    cu = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu[1:])
    kv_lens = np.asarray([s + q for s, q in zip(start_pos, q_lens)], dtype=np.int32)
    tables = []
    for gi in range(len(cache.kv_groups)):
        rows = cache.page_rows(gi, slots)
        width = max(1, max(len(r) for r in rows))
        tab = np.zeros((n, width), dtype=np.int32)
        for i, r in enumerate(rows):
            if r:
                tab[i, :len(r)] = np.maximum(np.asarray(r, dtype=np.int32), 0)
        tables.append(tab)
    pieces = [tokens, positions, seq_ids, cu, kv_lens, np.asarray(slots, dtype=np.int32),
              np.asarray(logit_rows, dtype=np.int32)] + [t.reshape(-1) for t in tables]
    flat = np.concatenate(pieces)
    host = torch.from_numpy(flat)
    if device.type == "cuda":
        host = host.pin_memory()
    dev = host.to(device, non_blocking=True)
    views, off = [], 0
    for p in pieces:
        views.append(dev[off:off + p.size])
        off += p.size
    ctx = StepContext(
        dtype=dtype, device=device, n_seqs=n, n_tokens=T, slots=list(slots), start_pos=list(start_pos),
        q_lens=q_lens, all_decode=all(q == 1 for q in q_lens), max_q_len=max(q_lens),
        max_kv_len=int(kv_lens.max()), tokens=views[0], positions=views[1], seq_ids=views[2], cu_seqlens=views[3],
        kv_lens=views[4], slots_dev=views[5],
        page_tables=[v.view(t.shape) for v, t in zip(views[7:], tables)])
    ctx.extras["host_buffer"] = host  # keep the pinned source alive until the copy has run
    rows = views[6] if logit_rows else None
    return ctx, rows


class StepFunction:
    """``step(inputs)`` -> float32 logits [number of wanted places, vocab] on the device, in the
    order of the inputs and of each input's ``want``."""

    def __init__(self, model, cache: SequenceCache, *, max_pass_tokens: int = 16384, max_sequence_chunk: int = 8192):
        self.model, self.cache = model, cache
        self.max_pass_tokens = max_pass_tokens
        self.max_sequence_chunk = max_sequence_chunk
        self.vocab_size = model.config.vocab_size

    def _validate(self, inputs: list[SequenceInput]) -> None:
        if not inputs:
            raise StepError("a step needs at least one sequence")
        seen = set()
        for i, s in enumerate(inputs):
            if s.slot in seen:
                raise StepError(f"slot {s.slot} appears twice in one step")
            seen.add(s.slot)
            if not self.cache.slots.is_live(s.slot):
                raise StepError(f"input {i}: slot {s.slot} is not live")
            if len(s.tokens) == 0:
                raise StepError(f"input {i}: no tokens")
            lo, hi = min(s.tokens), max(s.tokens)
            if lo < 0 or hi >= self.vocab_size:
                raise StepError(f"input {i}: token ids must be in [0, {self.vocab_size}), got {lo if lo < 0 else hi}")
            for w in s.want:
                if not (0 <= w < len(s.tokens)):
                    raise StepError(f"input {i}: wanted place {w} is outside its {len(s.tokens)} tokens")

    def __call__(self, inputs: list[SequenceInput]) -> torch.Tensor | None:
        self._validate(inputs)
        cache, model = self.cache, self.model
        # room for every token of the step is taken before anything is written
        cache.reserve([(s.slot, len(s.tokens)) for s in inputs])
        n_want = sum(len(s.want) for s in inputs)
        out_offsets, off = [], 0
        for s in inputs:
            out_offsets.append(off)
            off += len(s.want)

        total = sum(len(s.tokens) for s in inputs)
        longest = max(len(s.tokens) for s in inputs)
        if total <= self.max_pass_tokens and longest <= self.max_sequence_chunk:
            chunk = longest
        else:
            chunk = max(1, min(self.max_sequence_chunk, self.max_pass_tokens // len(inputs)))
            if chunk >= PAGE_TOKENS:
                chunk -= chunk % PAGE_TOKENS
        out = None
        done = 0
        while done < longest:
            part = [(i, s) for i, s in enumerate(inputs) if len(s.tokens) > done]
            slots = [s.slot for _, s in part]
            start = [cache.length(s.slot) for _, s in part]
            toks = [s.tokens[done:done + chunk] for _, s in part]
            rows, dest, base = [], [], 0
            for (i, s), t in zip(part, toks):
                for j, w in enumerate(s.want):
                    if done <= w < done + len(t):
                        rows.append(base + (w - done))
                        dest.append(out_offsets[i] + j)
                base += len(t)
            ctx, rows_dev = build_context(model.dtype, model.device, cache, slots, start, toks, rows)
            logits = model.forward(ctx, cache, rows_dev)
            for (_, s), t in zip(part, toks):
                cache.commit(s.slot, len(t))
            if logits is not None:
                if len(dest) == n_want and dest == list(range(n_want)):
                    out = logits
                else:
                    if out is None:
                        out = torch.empty((n_want, logits.shape[1]), dtype=torch.float32, device=logits.device)
                    out[torch.tensor(dest, device=logits.device)] = logits
            done += chunk
        return out
