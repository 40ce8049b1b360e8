"""Short prompts of one sequence as recorded passes: a prompt is padded with token 0 to the end of its last page,
run once as ordinary launches, recorded, and replayed for every later prompt of that size.

The padding must change nothing: not the logits of the real tokens (compared with the plain implementation, and bit
for bit between the first pass and its replays on other slots), not what later steps read (tokens decoded behind a
padded prompt, and a chunk appended behind one, are compared with the plain implementation too).  A model with a part
that does not say ``pad_safe`` is never run this way."""
import pytest
import torch

import plain_llama as P
from conftest import PEAKED, TINY, assert_close_logits, assert_within_plain_noise, make_model_dir, plain_inputs, random_prompts

pytestmark = pytest.mark.gpu


def _check(got, rows, ref, exact, dtype, what):
    """A handful of rows: float32 against the plain implementation; bfloat16 against its float64 run with the plain
    implementation's own rounding noise as the yardstick (the mean over so few numbers is no measure)."""
    if dtype == torch.float32:
        assert_close_logits(got, ref[rows], dtype, what)
    else:
        assert_within_plain_noise(got, exact[rows], ref[rows], dtype, what)


def _setup(session_tmp, name, dtype, max_tokens=4096):
    from gpullama3.java_b200.engine.step import StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    cfg_json, norm_std = TINY[name]
    d = make_model_dir(session_tmp, cfg_json, seed=23, norm_std=norm_std, scale=PEAKED)
    cfg, weights = plain_inputs(d)
    model = load_model(d, dtype)
    cache = model.new_cache(max_tokens)
    return cfg, weights, model, cache, StepFunction(model, cache)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_recorded_prompt_passes_and_what_follows_them(session_tmp, name, dtype):
    from gpullama3.java_b200.engine.step import SequenceInput

    cfg, weights, model, cache, step = _setup(session_tmp, name, dtype)
    assert step.use_prompt_graphs
    rt = None if dtype == torch.float32 else torch.bfloat16
    V = cfg["vocab_size"]
    recorded = set()                                                      # padded sizes that have a recording already
    for n in (5, 64, 65, 200, 640):
        seqs = random_prompts(V, [n + 4, n + 4, n + 4], seed=n)          # three prompts of one size: first pass, two replays
        refs = [P.forward(cfg, weights, s, round_to=rt) for s in seqs]
        exacts = [P.forward(cfg, weights, s, dtype=torch.float64) for s in seqs]
        replays = step.prompt_graph_replays
        firsts = []
        for k, (s, ref, exact) in enumerate(zip(seqs, refs, exacts)):
            slot = cache.acquire()
            if k == 2:                                                    # another slot and other pages than the recording's
                cache.release(slot)
                other = cache.acquire()
                slot = cache.acquire()
            got = step([SequenceInput(slot, s[:n], [0, n - 1])]).cpu()
            firsts.append(got)
            rows = [got] + [step([SequenceInput(slot, [s[j]], [0])]).cpu() for j in range(n, n + 4)]   # decoding behind the padding
            _check(torch.cat(rows), [0, n - 1, n, n + 1, n + 2, n + 3], ref, exact, dtype, f"tiny {name} prompt of {n}, pass {k}")
            cache.release(slot)
            if k == 2:
                cache.release(other)
        padded = -(-n // 64) * 64
        assert step.prompt_graph_replays == replays + (3 if padded in recorded else 2)
        recorded.add(padded)
        # the same prompt again, now replayed: the bits of its first pass (which ran as ordinary launches)
        slot = cache.acquire()
        again = step([SequenceInput(slot, seqs[0][:n], [0, n - 1])])
        assert torch.equal(again.cpu(), firsts[0])
        cache.release(slot)
    cache.check_invariants()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_a_chunk_behind_a_padded_prompt(session_tmp, dtype):
    """128 tokens (two whole pages), then 70 more as a pass of their own (padded to 128), then 3 one by one; and a
    prompt whose later chunk starts inside a page, which is not recorded."""
    from gpullama3.java_b200.engine.step import SequenceInput

    cfg, weights, model, cache, step = _setup(session_tmp, "B", dtype)
    rt = None if dtype == torch.float32 else torch.bfloat16
    s = random_prompts(cfg["vocab_size"], [128 + 70 + 3], seed=9)[0]
    ref = P.forward(cfg, weights, s, round_to=rt)
    exact = P.forward(cfg, weights, s, dtype=torch.float64)
    for rep in range(2):
        slot = cache.acquire()
        step([SequenceInput(slot, s[:128], [])])
        rows = [step([SequenceInput(slot, s[128:198], [0, 69])]).cpu()]
        rows += [step([SequenceInput(slot, [s[j]], [0])]).cpu() for j in range(198, 201)]
        _check(torch.cat(rows), [128, 197, 198, 199, 200], ref, exact, dtype, f"chunk behind two pages, run {rep}")
        cache.release(slot)
    assert step.prompt_graph_replays >= 2
    slot = cache.acquire()
    step([SequenceInput(slot, s[:100], [])])
    replays = step.prompt_graph_replays
    got = step([SequenceInput(slot, s[100:198], [0, 50, 97])])            # starts inside a page: ordinary launches
    _check(got.cpu(), [100, 150, 197], ref, exact, dtype, "chunk that starts inside a page")
    cache.release(slot)
    assert step.prompt_graph_replays == replays
    cache.check_invariants()


def test_a_part_that_is_not_pad_safe_keeps_the_model_off_recorded_prompts(session_tmp):
    from gpullama3.java_b200.engine.step import StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    cfg_json, norm_std = TINY["A"]
    d = make_model_dir(session_tmp, cfg_json, seed=23, norm_std=norm_std, scale=PEAKED)
    model = load_model(d, torch.bfloat16)
    assert model.pad_safe and model.graph_safe
    part = next(iter(model.named_parts().values()))
    part.pad_safe = False
    try:
        assert not model.pad_safe
        assert not StepFunction(model, model.new_cache(256)).use_prompt_graphs
    finally:
        del part.pad_safe


def test_recordings_are_kept_up_to_a_number_and_the_oldest_goes(session_tmp):
    from gpullama3.java_b200.engine.step import SequenceInput

    cfg, weights, model, cache, step = _setup(session_tmp, "A", torch.bfloat16)
    step.max_prompt_graphs = 2
    sizes = [10, 70, 130, 10, 70]            # padded 64, 128, 192: the third pushes the first out, the fourth records it again
    replays = []
    for n in sizes:
        slot = cache.acquire()
        p = random_prompts(cfg["vocab_size"], [n], seed=n)[0]
        got = step([SequenceInput(slot, p, [n - 1])])
        ref = P.forward(cfg, weights, p, round_to=torch.bfloat16)
        exact = P.forward(cfg, weights, p, dtype=torch.float64)
        _check(torch.cat([got.cpu(), got.cpu()]), [n - 1, n - 1], ref, exact, torch.bfloat16, f"prompt of {n}")
        cache.release(slot)
        replays.append(step.prompt_graph_replays)
        assert len(step._prompt_graphs) <= 2
    assert replays == [0, 0, 0, 0, 0]        # 64 was dropped when 192 came, 128 when 64 came back: nothing is replayed
    slot = cache.acquire()
    step([SequenceInput(slot, random_prompts(cfg["vocab_size"], [100], seed=1)[0], [])])   # padded 128, no wanted place: a new key
    step.max_prompt_graphs = 8
    cache.release(slot)
    slot = cache.acquire()
    step([SequenceInput(slot, random_prompts(cfg["vocab_size"], [70], seed=70)[0], [69])])  # 128 with one wanted place: still recorded
    cache.release(slot)
    assert step.prompt_graph_replays == 1
