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
from .workspace import Workspace


class StepError(ValueError):
    """The step was refused before anything ran (bad tokens, bad places, unknown slot)."""


@dataclass
class SequenceInput:
    slot: int
    tokens: list[int]
    want: list[int] = field(default_factory=list)  # places among ``tokens`` whose logits are wanted


def _pack(cache: SequenceCache, slots, start_pos, token_lists, logit_rows, widths=None):
    """The integer arrays of one pass, in the order they are laid out on the device."""
    n = len(slots)
    q_lens = [len(t) for t in token_lists]
    tokens = np.concatenate([np.asarray(t, dtype=np.int32) for t in token_lists])
    positions = np.concatenate([np.arange(s, s + q, dtype=np.int32) for s, q in zip(start_pos, q_lens)])
    seq_ids = np.repeat(np.arange(n, dtype=np.int32), q_lens)
    cu = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu[1:])
    kv_lens = np.asarray([s + q for s, q in zip(start_pos, q_lens)], dtype=np.int32)
    tables = []
    for gi in range(len(cache.paged_groups)):
        rows = cache.page_rows(gi, slots)
        width = widths[gi] if widths is not None else max(1, max(len(r) for r in rows))
        tab = np.zeros((n, width), dtype=np.int32)  # unused entries name page 0: never read, never out of range
        for i, r in enumerate(rows):
            if r:
                tab[i, :len(r)] = np.maximum(np.asarray(r, dtype=np.int32), 0)
        tables.append(tab)
    pieces = [tokens, positions, seq_ids, cu, kv_lens, np.asarray(slots, dtype=np.int32),
              np.asarray(logit_rows, dtype=np.int32)] + [t.reshape(-1) for t in tables]
    return pieces, q_lens, [t.shape for t in tables]


def _context_over(dev: torch.Tensor, sizes, table_shapes, dtype, device, slots, start_pos, q_lens, kv_capacity=None):
    views, off = [], 0
    for n in sizes:
        views.append(dev[off:off + n])
        off += n
    ctx = StepContext(
        dtype=dtype, device=device, n_seqs=len(slots), n_tokens=sum(q_lens), slots=list(slots),
        start_pos=list(start_pos), q_lens=list(q_lens), all_decode=all(q == 1 for q in q_lens), max_q_len=max(q_lens),
        max_kv_len=max(s + q for s, q in zip(start_pos, q_lens)), tokens=views[0], positions=views[1],
        seq_ids=views[2], cu_seqlens=views[3], kv_lens=views[4], slots_dev=views[5],
        page_tables=[v.view(shape) for v, shape in zip(views[7:], table_shapes)])
    ctx.kv_capacity = list(kv_capacity) if kv_capacity is not None else [ctx.max_kv_len] * len(table_shapes)
    return ctx, views[6]


def build_context(dtype, device, cache: SequenceCache, slots: list[int], start_pos: list[int],
                  token_lists: list, logit_rows: list[int], workspace=None) -> tuple[StepContext, torch.Tensor | None]:
    """Pack one pass into a StepContext.  All integers go to the device in one copy.  ``workspace``: where the
    pass takes its intermediate tensors from (it is reset here)."""
    pieces, q_lens, table_shapes = _pack(cache, slots, start_pos, token_lists, logit_rows)
    host = torch.from_numpy(np.concatenate(pieces))
    if device.type == "cuda":
        host = host.pin_memory()
    dev = host.to(device, non_blocking=True)
    ctx, rows = _context_over(dev, [p.size for p in pieces], table_shapes, dtype, device, slots, start_pos, q_lens)
    ctx.extras["host_buffer"] = host  # keep the pinned source alive until the copy has run
    if workspace is not None:
        workspace.reset()
        ctx.workspace = workspace
    return ctx, (rows if logit_rows else None)


def _record(launches):
    """Records ``launches()`` (which must have run once already as ordinary launches, so that every kernel library
    is loaded and configured) into a CUDA graph without running it; returns the graph, what ``launches`` returned
    inside the recording (tensors at fixed addresses) and the number of kernel launches recorded."""
    import gc

    from ..kernels import ops

    torch.cuda.synchronize()
    before = ops.launch_count()
    graph = torch.cuda.CUDAGraph()
    gc_was_on = gc.isenabled()
    gc.disable()  # a collection while recording could free device or pinned memory, which is not allowed then
    try:
        with torch.cuda.graph(graph):
            out = launches()
    finally:
        if gc_was_on:
            gc.enable()
    return graph, out, ops.launch_count() - before


class DecodeGraph:
    """One captured decode step for a fixed number of sequences and fixed page-table widths.

    Everything that changes from step to step (tokens, positions, lengths, page tables) lives in
    one device buffer at fixed addresses that is refreshed by a single copy before each replay, so
    the captured launch sequence is valid for any lengths the table widths can address.  The
    reference rebuilds nothing per token either: its plan is a list of pre-built task graphs
    replayed for every token (tornadovm/TornadoVMMasterPlan.java:149-175 of the reference
    project)."""

    def __init__(self, model, cache: SequenceCache, n_seqs: int, widths: list[int], sampler=None,
                 tokens_dev: torch.Tensor | None = None, fed: bool = False):
        """``tokens_dev``: where the draw leaves its tokens on the device (its own buffer if none is given).
        ``fed``: the step's input tokens are what ``tokens_dev`` holds when the step starts, i.e. the tokens the
        step before it drew for the same sequences; the host then stages positions and page tables only."""
        self.model, self.cache, self.n, self.widths = model, cache, n_seqs, list(widths)
        self.sampler = sampler                        # its launches are recorded after the model's, if given
        self.fed = bool(fed)
        assert not fed or (sampler is not None and tokens_dev is not None)
        self.draws = sampler is not None and sampler.uniforms([0], [0]) is not None
        self.sizes = [n_seqs, n_seqs, n_seqs, n_seqs + 1, n_seqs, n_seqs, n_seqs] + [n_seqs * w for w in widths]
        self.table_shapes = [(n_seqs, w) for w in widths]
        self.table_offsets, off = [], sum(self.sizes[:7])
        for w in widths:
            self.table_offsets.append(off)
            off += n_seqs * w
        self.uniform_offset = off                     # float32 numbers of the draws, after the integers
        total = off + (n_seqs if self.draws else 0)
        self.host = torch.empty(total, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.dev = torch.empty(total, dtype=torch.int32, device=model.device)
        if sampler is None:
            self.tokens_dev = None
        elif tokens_dev is not None:
            assert tokens_dev.shape == (n_seqs,) and tokens_dev.dtype == torch.int32
            self.tokens_dev = tokens_dev
        else:
            self.tokens_dev = torch.empty(n_seqs, dtype=torch.int32, device=model.device)
        self.tokens_host = torch.empty(n_seqs, dtype=torch.int32).pin_memory() if sampler is not None else None
        self.done = torch.cuda.Event()                # the last run of this step, copies included
        self.pending = False
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self.n_launches = 0
        self.h2d_bytes = total * 4
        self.d2h_bytes = n_seqs * 4 if sampler is not None else 0
        self.last_slots: list[int] | None = None
        self.last_pos: list[int] | None = None
        self.last_owners = -1                         # the cache's ownership count at the last refresh
        # the step is replayed for every length its page tables can address: parts shape their launches for that
        self.kv_capacity = [w * PAGE_TOKENS for w in widths]

    def refresh(self, slots, start_pos, tokens, uniforms=None) -> None:
        """Fill the staging buffer for this step.  A step that continues the one before (same slots, still the
        same sequences in them, every position one further) only rewrites what moved: tokens, positions,
        lengths, and the table row of a sequence that has just entered a new page."""
        if self.pending:
            self.done.synchronize()  # the run before must have read the staging buffer
            self.pending = False
        n, h = self.n, self.host_np
        owners = getattr(self.cache, "ownership_changes", None)
        if (self.last_slots == slots and owners is not None and owners == self.last_owners
                and all(q < p <= q + 2 for p, q in zip(start_pos, self.last_pos))):
            # (two further: this recorded step takes turns with another one)
            h[0:n] = tokens
            h[n:2 * n] = start_pos
            h[4 * n + 1:5 * n + 1] = h[n:2 * n] + 1
            for i, (p, q) in enumerate(zip(start_pos, self.last_pos)):
                if p // PAGE_TOKENS != q // PAGE_TOKENS:
                    for gi, (off, w) in enumerate(zip(self.table_offsets, self.widths)):
                        row = self.cache.page_rows(gi, [slots[i]])[0]
                        dst = h[off + i * w: off + (i + 1) * w]
                        dst[:len(row)] = np.maximum(np.asarray(row, dtype=np.int32), 0)
        else:
            pieces, _, _ = _pack(self.cache, slots, start_pos, [[t] for t in tokens], list(range(n)), self.widths)
            np.concatenate(pieces, out=h[:self.uniform_offset])
        if self.draws:
            h[self.uniform_offset:self.uniform_offset + n] = np.asarray(uniforms, dtype=np.float32).view(np.int32)
        self.last_slots, self.last_pos, self.last_owners = list(slots), list(start_pos), owners

    def _launches(self, slots, start_pos):
        """The step as it is issued and as it is recorded: staging buffer in, model, draw, tokens out."""
        self.dev.copy_(self.host, non_blocking=True)
        ctx, rows = _context_over(self.dev, self.sizes, self.table_shapes, self.model.dtype, self.model.device, slots,
                                  start_pos, [1] * self.n, self.kv_capacity)
        if self.fed:
            ctx.tokens = self.tokens_dev  # read by the embedding before this step's draw overwrites it
        logits = self.model.forward(ctx, self.cache, rows)
        if self.sampler is not None:
            u = self.dev[self.uniform_offset:self.uniform_offset + self.n].view(torch.float32) if self.draws else None
            self.sampler.sample_into(logits, u, self.tokens_dev)
            self.tokens_host.copy_(self.tokens_dev, non_blocking=True)
        return logits

    def run(self, slots, start_pos, tokens, uniforms=None, before_launch=None) -> torch.Tensor:
        """``before_launch``: called when the host side of the step is done, right before the step's first
        launch (a measurement records its start event there)."""
        self.refresh(slots, start_pos, tokens, uniforms)
        if before_launch is not None:
            before_launch()
        if self.graph is None:
            # the first step runs as ordinary launches (this also loads every kernel library the step
            # needs); the same launch sequence is then recorded, without running, for later steps
            out = self._launches(slots, start_pos)
            torch.cuda.synchronize()
            first_tokens = self.tokens_host.clone() if self.sampler is not None else None
            self.graph, self.logits, self.n_launches = _record(lambda: self._launches(slots, start_pos))
            if first_tokens is not None:
                self.tokens_host.copy_(first_tokens)
            return out
        self.graph.replay()
        self.done.record()
        self.pending = True
        return self.logits

    def sampled(self) -> list[int]:
        """The tokens drawn by the last run (waits for it)."""
        if self.pending:
            self.done.synchronize()
            self.pending = False
        return self.tokens_host.tolist()


class PromptGraph:
    """One recorded prompt pass of a single sequence: ``n_tokens`` tokens (a whole number of pages' worth), fixed
    page-table widths, a fixed number of wanted places.

    A prompt of a few hundred tokens is a hundred-odd launches that the GPU finishes sooner than the host can issue
    them; recorded once per size and replayed, the pass costs the host one copy and one launch.  A prompt is padded
    with token 0 up to the end of its last page: the padding runs as ordinary tokens of the pass (causal attention
    keeps it away from the real ones), writes keys and values into the part of that page no position has claimed
    yet, and is never committed to the cache, so later tokens overwrite it before anything reads it.  Only models
    whose parts all say ``pad_safe`` and ``graph_safe`` are run this way.  As in a recorded decode step, everything
    that changes from pass to pass lives in one device buffer refreshed by a single copy."""

    def __init__(self, model, cache: SequenceCache, n_tokens: int, widths: list[int], n_wanted: int):
        self.model, self.cache, self.n_tokens, self.widths, self.n_wanted = model, cache, n_tokens, list(widths), n_wanted
        self.sizes = [n_tokens, n_tokens, n_tokens, 2, 1, 1, n_wanted] + list(widths)
        self.table_shapes = [(1, w) for w in widths]
        total = sum(self.sizes)
        self.host = torch.empty(total, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.dev = torch.empty(total, dtype=torch.int32, device=model.device)
        self.done = torch.cuda.Event()
        self.pending = False
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self.n_launches = 0
        self.h2d_bytes = total * 4

    def _launches(self, slot: int, start: int):
        self.dev.copy_(self.host, non_blocking=True)
        ctx, rows = _context_over(self.dev, self.sizes, self.table_shapes, self.model.dtype, self.model.device, [slot],
                                  [start], [self.n_tokens])
        return self.model.forward(ctx, self.cache, rows if self.n_wanted else None)

    def run(self, slot: int, start: int, tokens: list[int], rows: list[int]) -> tuple[torch.Tensor | None, bool]:
        """Logits at ``rows`` (None when none are wanted) and whether the pass was replayed."""
        if self.pending:
            self.done.synchronize()  # the run before must have read the staging buffer
            self.pending = False
        padded = list(tokens) + [0] * (self.n_tokens - len(tokens))
        pieces, _, _ = _pack(self.cache, [slot], [start], [padded], rows, self.widths)
        np.concatenate(pieces, out=self.host_np)
        if self.graph is None:
            out = self._launches(slot, start)   # the first pass of this size runs as ordinary launches, then is recorded
            self.graph, self.logits, self.n_launches = _record(lambda: self._launches(slot, start))
            return out, False
        self.graph.replay()
        self.done.record()
        self.pending = True
        return (self.logits.clone() if self.logits is not None else None), True


class StepFunction:
    """``step(inputs)`` -> float32 logits [number of wanted places, vocab] on the device, in the
    order of the inputs and of each input's ``want``."""

    def __init__(self, model, cache: SequenceCache, *, max_pass_tokens: int = 16384, max_sequence_chunk: int = 8192,
                 use_graphs: bool = True, max_graph_batch: int = 256):
        self.model, self.cache = model, cache
        self.max_pass_tokens = max_pass_tokens
        self.max_sequence_chunk = max_sequence_chunk
        self.vocab_size = model.config.vocab_size
        # decode steps are replayed from CUDA graphs when every part says its launches do not depend on
        # host-side values of the step (parts default to "no": a part written without that in mind stays right)
        self.use_graphs = bool(use_graphs and model.device.type == "cuda" and getattr(model, "graph_safe", False))
        self.max_graph_batch = max_graph_batch
        self.reuse_output = False   # True: the caller consumes the logits before the next step (no copy is made)
        self._graphs: dict[tuple, DecodeGraph] = {}
        self.graph_launches = 0     # kernel launches replayed from graphs so far
        self.last_h2d_bytes = 0     # bytes of the last step's host-to-device copy (tokens, positions, page tables)
        self.last_d2h_bytes = 0     # bytes of the last step's copy of drawn tokens to the host (decode_and_sample)
        self.before_launch = None   # measurement hook: called between a recorded decode step's host work and its launch
        # short prompts of one sequence as recorded passes (PromptGraph), a few dozen sizes kept, the oldest dropped
        self.use_prompt_graphs = bool(self.use_graphs and getattr(model, "pad_safe", False))
        self.max_prompt_graph_tokens = 1024   # beyond this the GPU is the slower side and a recording saves nothing
        self.max_prompt_graphs = 32
        self._prompt_graphs: dict[tuple, PromptGraph] = {}
        self.prompt_graph_replays = 0
        self._drawn: dict[int, torch.Tensor] = {}   # per number of sequences: where every recorded draw leaves its tokens
        self._in_flight: list[DecodeGraph] = []     # steps launched by decode_ahead, oldest first, not yet collected
        self._fed_turn = 0
        # intermediate tensors of passes that are issued launch by launch (prompts, mixed steps); recorded decode
        # steps keep theirs in the graph's own memory
        self.workspace = Workspace(model.device) if model.device.type == "cuda" else None

    def _graph_for(self, slots: list[int], start: list[int], sampler=None, variant: int = 0) -> DecodeGraph:
        """The recorded step that fits these sequences: table widths are powers of two of at least 4 pages.
        ``variant`` 0 takes its tokens from the host; 1 and 2 are two copies of the step that takes them from the
        draw before it on the device (two, so that one can be staged while the other runs)."""
        cache = self.cache
        widths = []
        for gi in range(len(cache.paged_groups)):
            need = max(len(r) for r in cache.page_rows(gi, slots))
            w = 4
            while w < need:
                w *= 2
            widths.append(w)
        key = (len(slots), tuple(widths), sampler.launch_key() if sampler is not None else None, variant)
        g = self._graphs.get(key)
        if g is None:
            drawn = None
            if sampler is not None:
                drawn = self._drawn.get(len(slots))
                if drawn is None:
                    drawn = self._drawn[len(slots)] = torch.empty(len(slots), dtype=torch.int32, device=self.model.device)
            g = self._graphs[key] = DecodeGraph(self.model, cache, len(slots), widths, sampler, tokens_dev=drawn,
                                                fed=variant != 0)
        return g

    def decode_and_sample(self, inputs: list[SequenceInput], sampler, requests: list[int], draws: list[int]):
        """One token per sequence in, one drawn token per sequence out (host integers), as ONE recorded launch:
        staging copy, model, the sampler's kernels and the copy of the tokens back.  Returns None when the step
        cannot be served that way (graphs off, a part that is not graph-safe, too many sequences); the caller
        then takes the step and the sampler separately."""
        if self._in_flight:
            raise StepError("steps launched by decode_ahead have not been collected")
        if not self.decode_ahead(inputs, sampler, requests, draws):
            return None
        return self.collect()

    def decode_ahead(self, inputs: list[SequenceInput], sampler, requests: list[int], draws: list[int],
                     feed_previous: bool = False) -> bool:
        """Launch a decode step with its draw and return without waiting for the tokens; ``collect`` hands them
        out, oldest step first.  With ``feed_previous`` the step's input tokens are the ones the step launched
        just before it drew, taken on the device (the same sequences in the same order; the tokens in ``inputs``
        are placeholders): the host can launch step k + 1 while step k runs and read step k's tokens afterwards.
        Returns False, having done nothing, when the step cannot be served as a recorded launch."""
        if not (self.use_graphs and len(inputs) <= self.max_graph_batch and all(len(s.tokens) == 1 for s in inputs)
                and hasattr(sampler, "sample_into")):
            return False
        if len(self._in_flight) >= 2:
            raise StepError("two steps are in flight already: collect one first")
        self._validate(inputs)
        cache = self.cache
        slots = [s.slot for s in inputs]
        variant = 0
        if feed_previous:
            if not self._in_flight or self._in_flight[-1].last_slots != slots:
                raise StepError("feed_previous needs the step before, for the same sequences, to be in flight")
            self._fed_turn ^= 1
            variant = 1 + self._fed_turn
        cache.reserve([(s, 1) for s in slots])
        start = [cache.length(s) for s in slots]
        g = self._graph_for(slots, start, sampler, variant)
        if any(g is f for f in self._in_flight):  # cannot happen with two alternating copies; never stage under a running step
            raise StepError("the recorded step chosen is still in flight")
        replayed = g.graph is not None
        g.run(slots, start, [s.tokens[0] for s in inputs], sampler.uniforms(requests, draws), before_launch=self.before_launch)
        self.last_h2d_bytes, self.last_d2h_bytes = g.h2d_bytes, g.d2h_bytes
        if replayed:
            self.graph_launches += g.n_launches
        for s in slots:
            cache.commit(s, 1)
        self._in_flight.append(g)
        return True

    def collect(self) -> list[int]:
        """The tokens of the oldest step launched by ``decode_ahead`` and not collected yet (waits for it)."""
        if not self._in_flight:
            raise StepError("no step is in flight")
        return self._in_flight.pop(0).sampled()

    def abandon(self) -> None:
        """Forget the steps in flight (their tokens are not wanted any more; what they write into the cache
        lies in slots whose sequences are over)."""
        self._in_flight.clear()

    def _decode_with_graph(self, inputs: list[SequenceInput], reuse_output: bool) -> torch.Tensor | None:
        cache = self.cache
        n = len(inputs)
        slots = [s.slot for s in inputs]
        start = [cache.length(s) for s in slots]
        g = self._graph_for(slots, start)
        replayed = g.graph is not None
        logits = g.run(slots, start, [s.tokens[0] for s in inputs], before_launch=self.before_launch)
        self.last_h2d_bytes = g.h2d_bytes
        if replayed:
            self.graph_launches += g.n_launches
        for s in slots:
            cache.commit(s, 1)
        wanted = [i for i, s in enumerate(inputs) if s.want]
        if not wanted:
            return None
        if len(wanted) != n:
            return logits[torch.tensor(wanted, device=logits.device)]
        return logits if (reuse_output or not replayed) else logits.clone()

    def _prompt_with_graph(self, seq: SequenceInput):
        """The pass of one sequence's short prompt (or chunk) as a recorded pass; NotImplemented when it is not one
        for that: too long, too many wanted places, a start inside a page, or a size whose pages are not reserved."""
        cache = self.cache
        start, n = cache.length(seq.slot), len(seq.tokens)
        if n < 2 or n > self.max_prompt_graph_tokens or len(seq.want) > 8 or start % PAGE_TOKENS != 0:
            return NotImplemented
        padded = -(-n // PAGE_TOKENS) * PAGE_TOKENS          # up to the end of the last page the pass has reserved
        widths = []
        for gi in range(len(cache.paged_groups)):
            need = max(len(r) for r in cache.page_rows(gi, [seq.slot]))
            if need * PAGE_TOKENS < start + padded:
                return NotImplemented                        # (a group that keeps fewer pages than positions)
            w = 4
            while w < need:
                w *= 2
            widths.append(w)
        key = (padded, tuple(widths), len(seq.want))
        g = self._prompt_graphs.pop(key, None)
        if g is None:
            while len(self._prompt_graphs) >= self.max_prompt_graphs:
                self._prompt_graphs.pop(next(iter(self._prompt_graphs)))   # the one used longest ago
            g = PromptGraph(self.model, cache, padded, widths, len(seq.want))
        self._prompt_graphs[key] = g                          # (re-inserted: most recently used last)
        logits, replayed = g.run(seq.slot, start, seq.tokens, list(seq.want))
        self.last_h2d_bytes = g.h2d_bytes
        if replayed:
            self.prompt_graph_replays += 1
            self.graph_launches += g.n_launches
        cache.commit(seq.slot, n)
        return logits

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

    def __call__(self, inputs: list[SequenceInput], reuse_output: bool | None = None) -> torch.Tensor | None:
        """``reuse_output=True``: the caller is done with the returned logits before the next step (the
        tensor may be the fixed output buffer of a recorded decode step, which the next step overwrites)."""
        self._validate(inputs)
        cache, model = self.cache, self.model
        # room for every token of the step is taken before anything is written
        cache.reserve([(s.slot, len(s.tokens)) for s in inputs])
        if self.use_graphs and len(inputs) <= self.max_graph_batch and all(len(s.tokens) == 1 for s in inputs):
            return self._decode_with_graph(inputs, self.reuse_output if reuse_output is None else reuse_output)
        if self.use_prompt_graphs and len(inputs) == 1:
            out = self._prompt_with_graph(inputs[0])
            if out is not NotImplemented:
                return out
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
            ctx, rows_dev = build_context(model.dtype, model.device, cache, slots, start, toks, rows, self.workspace)
            self.last_h2d_bytes = ctx.extras["host_buffer"].numel() * 4
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
