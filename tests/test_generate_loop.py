"""The generation loop's decisions, with a scripted step function on the CPU (no GPU): batching,
stop tokens, sequences that end earlier, slot reuse, limits."""
import pytest
import torch

from gpullama3.java_b200.cache import KVCacheNeed, SequenceCache
from gpullama3.java_b200.engine.generate import (FINISH_CONTEXT, FINISH_LENGTH, FINISH_STOP, GenerationError,
                                                 Generator, plan_batches)
from gpullama3.java_b200.sampling import SamplingParams, uniform

VOCAB = 50


class ScriptedStep:
    """Stands in for the model: the 'logits' of a sequence point at (sum of its tokens) % VOCAB.
    It keeps the cache's lengths as the real step function does and records every call."""

    def __init__(self, cache):
        self.cache, self.calls, self.sums = cache, [], {}

    def __call__(self, inputs):
        self.cache.reserve([(s.slot, len(s.tokens)) for s in inputs])
        rows = []
        for s in inputs:
            if self.cache.length(s.slot) == 0:
                self.sums[s.slot] = 0
            self.sums[s.slot] += sum(s.tokens)
            self.cache.commit(s.slot, len(s.tokens))
            assert s.want == [len(s.tokens) - 1]
            row = torch.zeros(VOCAB)
            row[self.sums[s.slot] % VOCAB] = 1.0
            rows.append(row)
        self.calls.append([(s.slot, len(s.tokens)) for s in inputs])
        return torch.stack(rows)


class ArgmaxSampler:
    def __init__(self, params):
        self.params = params

    def sample(self, logits, requests, draws):
        self.last = (list(requests), list(draws))
        return logits.argmax(dim=-1).tolist()


def make(max_tokens=64 * 8, max_batch=4, max_length=None):
    cache = SequenceCache({0: KVCacheNeed(1, 16)}, max_tokens=max_tokens, max_slots=max_batch, dtype=torch.float32,
                          device="cpu")
    step = ScriptedStep(cache)
    gen = Generator(step, cache, ArgmaxSampler, max_batch=max_batch, max_length=max_length or max_tokens)
    return gen, step, cache


def expected_tokens(prompt, n, stop=()):
    out, s = [], sum(prompt)
    for _ in range(n):
        t = s % VOCAB
        out.append(t)
        s += t
        if t in stop:
            break
    return out


def test_unequal_prompts_one_step_then_one_token_each():
    gen, step, cache = make()
    prompts = [[1, 2, 3], [4] * 11, [5] * 17]
    res = gen.generate(prompts, 4, SamplingParams())
    assert [r.tokens for r in res] == [expected_tokens(p, 4) for p in prompts]
    assert all(r.finish_reason == FINISH_LENGTH for r in res)
    assert sorted(n for _, n in step.calls[0]) == [3, 11, 17]            # all prompts in one step
    assert all(n == 1 for call in step.calls[1:] for _, n in call)       # then one token each
    assert len(step.calls) == 4                                          # the 4th token is not fed back
    assert cache.live_slots() == [] and cache.paged_groups[0].pool.n_held == 0
    m = gen.last_metrics
    assert (m.prompt_tokens, m.generated_tokens, m.decode_steps) == (31, 12, 3)


def test_stop_token_is_kept_and_ends_only_its_sequence():
    gen, step, cache = make()
    prompts = [[7], [1, 2]]
    free_run = [expected_tokens(p, 6) for p in prompts]
    stop = {free_run[0][2]} - set(free_run[1])       # a token the first request produces third
    assert stop
    res = gen.generate(prompts, 6, SamplingParams(), stop_ids=stop)
    assert res[0].tokens == free_run[0][:3] and res[0].finish_reason == FINISH_STOP
    assert res[1].tokens == free_run[1] and res[1].finish_reason == FINISH_LENGTH
    sizes = [len(c) for c in step.calls]
    assert sizes == [2, 2, 2, 1, 1, 1]               # the batch shrinks when the first request ends


def test_batches_follow_one_another_and_use_slots_again():
    gen, step, cache = make(max_batch=2)
    prompts = [[i + 1] * (i + 1) for i in range(5)]
    res = gen.generate(prompts, 3, SamplingParams())
    assert [r.tokens for r in res] == [expected_tokens(p, 3) for p in prompts]
    firsts = [c for c in step.calls if any(n > 1 for _, n in c) or c == [(0, 1)]]
    used_slots = {s for c in step.calls for s, _ in c}
    assert used_slots <= {0, 1}                      # five requests through two slots
    assert cache.live_slots() == []


def test_plan_batches_respects_batch_size_and_pages():
    assert plan_batches([10, 10, 10, 10, 10], 5, 2, 100, 1000) == [[0, 1], [2, 3], [4]]
    # 3 pages in the cache; requests need 1, 2, 1, 3 pages at their longest
    assert plan_batches([10, 70, 10, 129], 20, 8, 3, 1000) == [[0, 1], [2], [3]]
    with pytest.raises(GenerationError, match="cache pages"):
        plan_batches([300], 10, 8, 3, 1000)
    with pytest.raises(GenerationError, match="empty"):
        plan_batches([0], 10, 8, 3, 1000)
    with pytest.raises(GenerationError, match="longest"):
        plan_batches([50], 10, 8, 3, 40)


def test_context_limit_ends_a_sequence():
    gen, step, cache = make(max_length=6)
    res = gen.generate([[1, 2, 3, 4]], 10, SamplingParams())
    assert res[0].finish_reason == FINISH_CONTEXT and len(res[0].tokens) == 2   # 4 + 2 = 6 positions


def test_slots_are_released_when_a_step_fails():
    gen, step, cache = make()

    def boom(inputs):
        raise RuntimeError("device fell over")
    gen.step_fn = boom
    with pytest.raises(RuntimeError):
        gen.generate([[1], [2]], 3, SamplingParams())
    assert cache.live_slots() == [] and cache.slots.n_free == 4


def test_sampler_sees_request_ids_and_draw_indices():
    gen, step, cache = make(max_batch=2)
    samplers = []

    def factory(p):
        samplers.append(ArgmaxSampler(p))
        return samplers[-1]
    gen.sampler_factory = factory
    gen.generate([[1], [2], [3]], 2, SamplingParams(temperature=0.5, seed=3), request_ids=[10, 11, 12])
    assert samplers[0].params.seed == 3
    assert samplers[0].last == ([12], [1])           # last call: third request, its second draw


def test_zero_new_tokens_runs_nothing():
    gen, step, cache = make()
    res = gen.generate([[1, 2]], 0, SamplingParams())
    assert res[0].tokens == [] and step.calls == []


def test_uniform_numbers_depend_only_on_their_arguments():
    a = [uniform(1, r, d) for r in range(4) for d in range(50)]
    assert all(0.0 <= x < 1.0 for x in a) and len(set(a)) == len(a)
    assert uniform(1, 2, 3) == uniform(1, 2, 3) != uniform(2, 2, 3)
    assert all(float(torch.tensor(x, dtype=torch.float32)) == x for x in a)   # exact in float32
    assert 0.4 < sum(a) / len(a) < 0.6


def test_sampling_params_are_validated_like_the_reference():
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1)
    with pytest.raises(ValueError):
        SamplingParams(top_p=1.5)
    assert SamplingParams().greedy and not SamplingParams(temperature=0.1).greedy


def test_decode_steps_go_to_the_step_and_draw_call_when_it_is_offered():
    """A step function may offer ``decode_and_sample`` (one call that runs a decode step and draws the tokens);
    the loop then uses it for every decode step, passes it the draws' identities, and falls back to step-then-
    sample for the steps it declines (returns None).  The prompt step is always sampled by the sampler."""
    gen, step, cache = make()
    fused_calls = []

    def decode_and_sample(inputs, sampler, requests, draws):
        if len(fused_calls) % 2 == 1:          # decline every other step
            fused_calls.append(None)
            return None
        logits = step(inputs)
        fused_calls.append((list(requests), list(draws)))
        return logits.argmax(dim=-1).tolist()

    step.decode_and_sample = decode_and_sample
    prompts = [[1, 2, 3], [4] * 11]
    res = gen.generate(prompts, 5, SamplingParams(), request_ids=[7, 9])
    assert [r.tokens for r in res] == [expected_tokens(p, 5) for p in prompts]
    assert len(fused_calls) == 4 and fused_calls[1] is None and fused_calls[3] is None
    assert fused_calls[0] == ([7, 9], [1, 1]) and fused_calls[2] == ([7, 9], [3, 3])
    assert cache.live_slots() == []


class AheadStep(ScriptedStep):
    """A scripted step function that also offers ``decode_ahead`` / ``collect`` / ``abandon`` the way the real
    one does: a launched step computes at once here, but its tokens stay "on the device" (``self.drawn``) until
    collected, and a step launched with ``feed_previous`` takes its input from there, not from the host."""

    def __init__(self, cache, decline=lambda n: False):
        super().__init__(cache)
        self.in_flight, self.drawn, self.drawn_slots = [], None, None
        self.launches, self.decline = [], decline

    def decode_ahead(self, inputs, sampler, requests, draws, feed_previous=False):
        if self.decline(len(self.launches)):
            assert not feed_previous, "a declined launch ahead would leave the loop without its tokens"
            return False
        assert len(self.in_flight) < 2
        slots = [s.slot for s in inputs]
        if feed_previous:
            assert self.in_flight and self.drawn_slots == slots, "fed from a step for other sequences"
            assert all(s.tokens == [0] for s in inputs), "the host does not know these tokens yet"
            inputs = [type(s)(s.slot, [t], [0]) for s, t in zip(inputs, self.drawn)]
        logits = self(inputs)
        self.drawn, self.drawn_slots = logits.argmax(dim=-1).tolist(), slots
        self.in_flight.append(list(self.drawn))
        self.launches.append((bool(feed_previous), list(requests), list(draws)))
        return True

    def collect(self):
        return self.in_flight.pop(0)

    def abandon(self):
        self.in_flight.clear()


def make_ahead(decline=lambda n: False, **kw):
    gen, _, cache = make(**kw)
    step = AheadStep(cache, decline)
    gen.step_fn = step
    return gen, step, cache


def test_steps_launched_one_ahead_give_the_same_tokens():
    """With ``decode_ahead`` the loop launches step k + 1 before it has read step k's tokens.  Results, finish
    reasons and the draws' identities are those of the plain loop, for stop tokens at every place, unequal
    lengths, length and context limits, and one batch after another."""
    import random
    rng = random.Random(5)
    for trial in range(60):
        n = rng.randint(1, 6)
        prompts = [[rng.randrange(1, VOCAB) for _ in range(rng.randint(1, 40))] for _ in range(n)]
        new = rng.randint(1, 12)
        stop = frozenset(rng.sample(range(VOCAB), rng.randint(0, 12)))
        max_length = rng.choice([None, 45])
        plain, _, _ = make(max_batch=3, max_length=max_length)
        want = plain.generate(prompts, new, SamplingParams(), stop_ids=stop)
        seen = []
        gen, step, cache = make_ahead(max_batch=3, max_length=max_length)
        got = gen.generate(prompts, new, SamplingParams(), stop_ids=stop, on_token=lambda i, t: seen.append((i, t)))
        assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in want], trial
        assert sorted(seen) == sorted((i, t) for i, r in enumerate(want) for t in r.tokens)
        assert step.in_flight == [] and cache.live_slots() == [] and cache.paged_groups[0].pool.n_held == 0
        # token number d of a request (counting from 0, the prompt step's) was drawn as its draw d; a step launched
        # ahead may have drawn one more for a request that a stop token had just ended, and nothing beyond that
        drawn = {}
        for fed, requests, draws in step.launches:
            assert len(requests) == len(draws)
            for r, d in zip(requests, draws):
                assert d not in drawn.setdefault(r, set()), "a draw was made twice"
                drawn[r].add(d)
        for i, r in enumerate(want):
            made = drawn.get(i, set())
            kept = set(range(1, len(r.tokens)))
            extra = made - kept
            assert kept <= made and extra <= ({len(r.tokens)} if r.finish_reason == FINISH_STOP else set()), (trial, i)
        assert gen.last_metrics.generated_tokens == sum(len(r.tokens) for r in want)


def test_a_stop_token_drops_what_was_launched_ahead_for_its_sequence_only():
    gen, step, cache = make_ahead()
    prompts = [[1, 2, 3], [4] * 11]
    first = expected_tokens(prompts[0], 8)
    stop = {first[2]}                                    # sequence 0 ends with its third token
    assert first[2] not in expected_tokens(prompts[1], 8)
    res = gen.generate(prompts, 8, SamplingParams(), stop_ids=stop, request_ids=[7, 9])
    assert res[0].tokens == first[:3] and res[0].finish_reason == FINISH_STOP
    assert res[1].tokens == expected_tokens(prompts[1], 8) and res[1].finish_reason == FINISH_LENGTH
    # token 1 comes from the prompts; steps for tokens 2, 3 and (launched ahead, dropped for sequence 0) 4 hold both
    # sequences, the first from host tokens, the others fed on the device; then sequence 1 goes on alone
    assert step.launches[0] == (False, [7, 9], [1, 1])
    assert step.launches[1] == (True, [7, 9], [2, 2]) and step.launches[2] == (True, [7, 9], [3, 3])
    assert step.launches[3] == (False, [9], [4]) and all(l[1] == [9] for l in step.launches[3:])
    assert [l[2] for l in step.launches[3:]] == [[4], [5], [6], [7]]
    assert [l[0] for l in step.launches[3:]] == [False, True, True, True]
    assert gen.last_metrics.decode_steps == len(step.launches)


def test_nothing_is_launched_past_a_limit_that_is_known_beforehand():
    """The last token of a sequence that ends by length or by the context limit is known to be its last before
    it is drawn: no step is launched ahead for it, so the cache never holds a position past the plan."""
    gen, step, cache = make_ahead(max_length=14)
    res = gen.generate([[1, 2, 3], [4] * 11], 6, SamplingParams())
    assert [len(r.tokens) for r in res] == [6, 3] and [r.finish_reason for r in res] == [FINISH_LENGTH, FINISH_CONTEXT]
    per_slot = {}
    for call in step.calls:
        for slot, n in call:
            per_slot[slot] = per_slot.get(slot, 0) + n
    assert sorted(per_slot.values()) == [3 + 5, 11 + 2]  # every token but the last is fed back, none beyond


def test_a_step_function_that_declines_is_served_the_plain_way():
    gen, step, cache = make_ahead(decline=lambda n: True)
    prompts = [[1, 2, 3], [4] * 11]
    res = gen.generate(prompts, 5, SamplingParams())
    assert [r.tokens for r in res] == [expected_tokens(p, 5) for p in prompts] and step.launches == []


def test_steps_in_flight_are_forgotten_when_the_loop_fails():
    gen, step, cache = make_ahead()

    def boom(i, tok):
        if len(step.launches) >= 2:
            raise RuntimeError("callback failed")

    with pytest.raises(RuntimeError):
        gen.generate([[1, 2, 3]], 8, SamplingParams(), on_token=boom)
    assert step.in_flight == [] and cache.live_slots() == []
    res = gen.generate([[1, 2, 3]], 4, SamplingParams())   # the next request is not served a stale step's tokens
    assert res[0].tokens == expected_tokens([1, 2, 3], 4)


def test_generation_stops_at_the_configurations_context_length():
    """The longest sequence is the smaller of what the cache holds and the configuration's own context length (the
    reference caps every run at it, inference/InferenceEngine.java:75-77 of the reference project); an explicit
    limit wins.  A prompt beyond it is refused, and a sequence that reaches it ends with the reason "context"."""
    from conftest import TINY_A
    from gpullama3.java_b200.config import config_from_dict
    from gpullama3.java_b200.engine.api import resolve_max_length
    from gpullama3.java_b200.engine.generate import FINISH_CONTEXT

    cfg = config_from_dict(dict(TINY_A, max_position_embeddings=20))
    assert resolve_max_length(cfg, 64 * 8) == 20
    assert resolve_max_length(cfg, 16) == 16
    assert resolve_max_length(cfg, 64 * 8, asked=300) == 300
    with pytest.raises(ValueError):
        resolve_max_length(cfg, 64, asked=0)
    gen, step, cache = make(max_length=resolve_max_length(cfg, 64 * 8))
    with pytest.raises(GenerationError, match="exceeds the longest sequence"):
        gen.generate([[1] * 21], 4, SamplingParams())
    res = gen.generate([[1] * 17, [2] * 3], 10, SamplingParams())
    assert res[0].finish_reason == FINISH_CONTEXT and len(res[0].tokens) == 3     # 17 + 3 = 20 positions
    assert res[1].finish_reason == FINISH_LENGTH and len(res[1].tokens) == 10
    assert cache.live_slots() == []


def test_span_rule_of_decode_attention():
    """How many spans a decode step cuts its keys into: one wave of CTAs at most, up to 16 spans of at least two
    blocks of 32 keys, beyond that at least 8 blocks a span, always a power of two."""
    from gpullama3.java_b200.kernels.ops import attention_decode_splits as splits

    assert splits(1, 8, 4096, 592) == 16        # batch 1 at 4,096 keys: 16 spans, not the 64 the GPU would hold
    assert splits(1, 8, 1024, 592) == 16        # a short context still gets spans of two blocks
    assert splits(1, 8, 16384, 592) == 64       # long rows: 8 blocks a span, 64 spans at most
    assert splits(8, 8, 4096, 592) == 8         # batch 8: 9 would fit one wave, 8 is the power of two
    assert splits(8, 8, 512, 592) == 8
    assert splits(64, 8, 4096, 592) == 1        # the batch alone fills the GPU
    assert splits(1, 8, 40, 592) == 1           # one block of keys
    for args in [(3, 4, 777, 592), (1, 1, 100000, 296), (200, 8, 64, 592)]:
        s = splits(*args)
        assert s >= 1 and s & (s - 1) == 0 and s * args[0] * args[1] <= max(args[3], args[0] * args[1])
