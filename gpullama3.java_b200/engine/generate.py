"""The generation loop above the step function: batches of unequal prompts, stop tokens,
sequences that end earlier, and as many batches one after another as there are requests.

One batch follows inference/InferenceEngine.java:309-355 of the reference project for each of its
sequences: the prompt goes in (here in one step, there token by token), then one token is sampled
per step from the sequence's own logits, recorded, and checked against the stop tokens; the stop
token is part of the result (:346-348).  A sequence that ends leaves the batch; the others go on.
When the batch ends its slots are given back and the next batch uses them again."""
from __future__ import annotations

import time
from dataclasses import dataclass, field

from ..cache.pages import pages_for
from .step import SequenceInput

FINISH_STOP = "stop"          # a stop token was sampled (it is the last token of the result)
FINISH_LENGTH = "length"      # max_new_tokens were generated
FINISH_CONTEXT = "context"    # the sequence reached the longest length the engine allows


@dataclass
class GenerationResult:
    prompt_length: int
    tokens: list[int] = field(default_factory=list)
    finish_reason: str | None = None


@dataclass
class RunMetrics:
    """What the reference's LastRunMetrics reports (auxiliary/LastRunMetrics.java:20-32: prompt +
    generated tokens over the wall time of the loop), with prefill and decode told apart."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    seconds: float = 0.0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    decode_steps: int = 0

    @property
    def tokens_per_second(self) -> float:
        return (self.prompt_tokens + self.generated_tokens) / self.seconds if self.seconds > 0 else 0.0


class GenerationError(ValueError):
    pass


def plan_batches(prompt_lengths: list[int], max_new_tokens: int, max_batch: int, n_pages: int,
                 max_length: int) -> list[list[int]]:
    """Cut the requests, in order, into batches: at most ``max_batch`` sequences each, and the pages
    of every sequence at its longest (prompt + max_new_tokens, capped by ``max_length``) must fit
    the cache together, so that no batch can run out of pages half-way."""
    batches, cur, cur_pages = [], [], 0
    for i, n in enumerate(prompt_lengths):
        if n < 1:
            raise GenerationError(f"request {i}: empty prompt")
        if n > max_length:
            raise GenerationError(f"request {i}: prompt of {n} tokens exceeds the longest sequence allowed ({max_length})")
        need = pages_for(min(n + max_new_tokens, max_length))
        if need > n_pages:
            raise GenerationError(f"request {i}: needs {need} cache pages, the cache has {n_pages}")
        if cur and (len(cur) >= max_batch or cur_pages + need > n_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += need
    if cur:
        batches.append(cur)
    return batches


class Generator:
    """``step_fn(inputs) -> logits rows``; ``sampler.sample(logits, requests, draws) -> tokens``;
    ``cache`` gives ``acquire``/``release`` and the number of pages."""

    def __init__(self, step_fn, cache, sampler_factory, *, max_batch: int, max_length: int):
        self.step_fn, self.cache, self.sampler_factory = step_fn, cache, sampler_factory
        self.max_batch, self.max_length = max_batch, max_length
        self.last_metrics = RunMetrics()

    def generate(self, prompts: list[list[int]], max_new_tokens: int, sampling, stop_ids=(), on_token=None,
                 request_ids: list[int] | None = None) -> list[GenerationResult]:
        """Generate for every prompt; results come back in the order of the prompts.
        ``on_token(request_index, token)`` is called for every sampled token as it is produced."""
        stop = frozenset(stop_ids)
        results = [GenerationResult(len(p)) for p in prompts]
        ids = request_ids if request_ids is not None else list(range(len(prompts)))
        metrics = RunMetrics()
        t_start = time.perf_counter()
        if max_new_tokens <= 0:
            for r in results:
                r.finish_reason = FINISH_LENGTH
            self.last_metrics = metrics
            return results
        sampler = self.sampler_factory(sampling)
        n_pages = self.cache.pages_for_planning()
        for batch in plan_batches([len(p) for p in prompts], max_new_tokens, min(self.max_batch, self.cache.max_slots),
                                  n_pages, self.max_length):
            slots = {i: self.cache.acquire() for i in batch}
            try:
                self._run_batch(batch, slots, prompts, results, ids, max_new_tokens, sampler, stop, on_token, metrics)
            finally:
                abandon = getattr(self.step_fn, "abandon", None)
                if abandon is not None:
                    abandon()  # after an error a step may still be in flight; its tokens belong to no one
                for s in slots.values():
                    self.cache.release(s)
        metrics.seconds = time.perf_counter() - t_start
        self.last_metrics = metrics
        return results

    def _run_batch(self, batch, slots, prompts, results, ids, max_new_tokens, sampler, stop, on_token, metrics):
        t0 = time.perf_counter()
        live = list(batch)
        inputs = [SequenceInput(slots[i], list(prompts[i]), [len(prompts[i]) - 1]) for i in live]
        logits = self.step_fn(inputs)
        metrics.prompt_tokens += sum(len(prompts[i]) for i in live)
        tokens = sampler.sample(logits, [ids[i] for i in live], [len(results[i].tokens) for i in live])
        metrics.prefill_seconds += time.perf_counter() - t0
        t0 = time.perf_counter()

        def take(who, toks):
            """Record one new token for each sequence of ``who``; returns the sequences that go on."""
            nxt = []
            for i, tok in zip(who, toks):
                r = results[i]
                r.tokens.append(tok)
                metrics.generated_tokens += 1
                if on_token is not None:
                    on_token(i, tok)
                if tok in stop:
                    r.finish_reason = FINISH_STOP
                elif len(r.tokens) >= max_new_tokens:
                    r.finish_reason = FINISH_LENGTH
                elif r.prompt_length + len(r.tokens) >= self.max_length:
                    r.finish_reason = FINISH_CONTEXT  # no room to feed the token back
                else:
                    nxt.append(i)
            return nxt

        def goes_on_unless_it_stops(i):
            """Whether sequence i, with the token of the step in flight still to come, has room for one more."""
            r = results[i]
            return len(r.tokens) + 1 < max_new_tokens and r.prompt_length + len(r.tokens) + 1 < self.max_length

        fused = getattr(self.step_fn, "decode_and_sample", None)  # step and draw as one recorded launch, if offered
        ahead = getattr(self.step_fn, "decode_ahead", None)       # the same without waiting for the tokens
        collect = getattr(self.step_fn, "collect", None)
        if collect is None:
            ahead = None
        live = take(live, tokens)
        while live:
            inputs = [SequenceInput(slots[i], [results[i].tokens[-1]], [0]) for i in live]
            requests, draws = [ids[i] for i in live], [len(results[i].tokens) for i in live]
            metrics.decode_steps += 1
            if ahead is None or not ahead(inputs, sampler, requests, draws, False):
                tokens = fused(inputs, sampler, requests, draws) if fused is not None else None
                if tokens is None:
                    tokens = sampler.sample(self.step_fn(inputs), requests, draws)
                live = take(live, tokens)
                continue
            # A step is in flight.  While it runs, the step after it is launched for the same sequences, fed with
            # the tokens of the step in flight on the device; the host reads tokens one step late.  Only a stop
            # token can end a sequence unforeseen: the token the step launched ahead drew for it is dropped (what
            # that step wrote into the cache lies behind the sequence's end), and the batch goes on without it.
            while True:
                placeholders = [SequenceInput(slots[i], [0], [0]) for i in live]
                launched_ahead = (all(goes_on_unless_it_stops(i) for i in live)
                                  and ahead(placeholders, sampler, requests, [len(results[i].tokens) + 1 for i in live], True))
                nxt = take(live, collect())
                if not launched_ahead:
                    live = nxt
                    break
                metrics.decode_steps += 1
                if nxt == live:
                    continue
                going = set(nxt)
                pairs = [(i, tok) for i, tok in zip(live, collect()) if i in going]
                live = take([i for i, _ in pairs], [tok for _, tok in pairs])
                break
        metrics.decode_seconds += time.perf_counter() - t0
