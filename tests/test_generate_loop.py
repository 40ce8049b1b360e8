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
    assert cache.live_slots() == [] and cache.kv_groups[0].pool.n_held == 0
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
