"""Replay of the same requests cut in different ways: whole, with the last 32 tokens decoded one by
one, and in batches of unequal lengths whose shorter requests end earlier, one batch after another
with a cache so small that slots and pages are used again.  Every way must give the plain
implementation's logits at every position that is asked for.  The weights make attention peaked,
so one wrong key, position or cache page shows."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_llama
from conftest import PEAKED, ROOT, TINY, assert_close_logits, make_model_dir, plain_inputs, random_prompts
from replay_helpers import (max_live_tokens, read_rows, run_in_process, trace_batches, trace_tail_one_by_one,
                            trace_whole, write_trace)

pytestmark = pytest.mark.gpu

LENGTHS = [33, 64, 65, 100, 129, 40, 200, 70]


def _reference(cfg, weights, requests, dtype):
    rt = None if dtype == torch.float32 else torch.bfloat16
    return {rid: plain_llama.forward(cfg, weights, toks, round_to=rt) for rid, toks in requests.items()}


def _check(got, ref, dtype, what):
    by_req: dict = {}
    for (rid, pos), row in got.items():
        by_req.setdefault(rid, []).append((pos, row))
    for rid, items in by_req.items():
        items.sort()
        g = torch.stack([r for _, r in items])
        r = ref[rid][[p for p, _ in items]]
        assert_close_logits(g, r, dtype, f"{what} request {rid}")


@pytest.fixture(scope="module", params=["A", "B"])
def setup(request, session_tmp):
    cfg_json, norm_std = TINY[request.param]
    d = make_model_dir(session_tmp, cfg_json, seed=3, norm_std=norm_std, scale=PEAKED)
    cfg, weights = plain_inputs(d)
    prompts = random_prompts(cfg["vocab_size"], LENGTHS, seed=11)
    requests = {f"r{i}": p for i, p in enumerate(prompts)}
    refs = {}
    return d, cfg, weights, requests, refs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("cut", ["whole", "tail32", "batches3", "batches8"])
def test_replay_cuts_match_plain(setup, tmp_path, dtype, cut):
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, weights, requests, refs = setup
    if dtype not in refs:
        refs[dtype] = _reference(cfg, weights, requests, dtype)
    if cut == "whole":
        steps, rows = trace_whole(requests)
    elif cut == "tail32":
        steps, rows = trace_tail_one_by_one(requests, 32)
    elif cut == "batches3":
        steps, rows = trace_batches(requests, 3)
    else:
        steps, rows = trace_batches(requests, 8, prompt_fraction=0.3)
    model = load_model(d, dtype)
    run_in_process(model, steps, tmp_path, max_live_tokens(steps))  # the smallest cache the trace is promised
    got = read_rows(tmp_path, rows, cfg["vocab_size"])
    _check(got, refs[dtype], dtype, cut)


def test_trace_run_program(setup, tmp_path):
    """The program itself, as a user starts it: steps on standard input, 'done <step>' lines out."""
    d, cfg, weights, requests, refs = setup
    few = dict(list(requests.items())[:4])
    steps, rows = trace_batches(few, 2)
    trace = tmp_path / "trace.jsonl"
    write_trace(trace, steps)
    out = tmp_path / "out"
    env = dict(os.environ, PYTHON=sys.executable)
    with open(trace) as f:
        p = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out),
                            "--max-tokens", str(max_live_tokens(steps))], stdin=f, capture_output=True, text=True,
                           env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    got = read_rows(out, rows, cfg["vocab_size"])
    _check(got, _reference(cfg, weights, few, torch.float32), torch.float32, "trace_run")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_a_step_cut_into_passes_gives_the_same_logits(setup, dtype):
    """A step with more tokens than one pass may hold is run as several passes (chunks of each sequence
    that continue what the earlier pass cached); wanted places of all passes come back in the order asked."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, weights, requests, refs = setup
    if dtype not in refs:
        refs[dtype] = _reference(cfg, weights, requests, dtype)
    model = load_model(d, dtype)
    cache = model.new_cache(64 * 16)
    ids = list(requests)[:5]
    wants = {r: sorted({0, len(requests[r]) // 3, len(requests[r]) - 1}) for r in ids}
    for limits in (dict(max_pass_tokens=96, max_sequence_chunk=8192), dict(max_pass_tokens=16384, max_sequence_chunk=40)):
        step = StepFunction(model, cache, **limits)
        slots = {r: cache.acquire() for r in ids}
        out = step([SequenceInput(slots[r], requests[r], wants[r]) for r in ids]).cpu()
        off = 0
        for r in ids:
            n = len(wants[r])
            assert_close_logits(out[off:off + n], refs[dtype][r][wants[r]], dtype, f"passes {limits} request {r}")
            off += n
        for r in ids:
            assert cache.length(slots[r]) == len(requests[r])
            cache.release(slots[r])
    cache.check_invariants()


def test_a_step_that_does_not_fit_changes_nothing(setup):
    from gpullama3.java_b200.cache import CacheFull
    from gpullama3.java_b200.engine.step import SequenceInput, StepError, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, weights, requests, refs = setup
    model = load_model(d, torch.float32)
    cache = model.new_cache(64 * 3)
    step = StepFunction(model, cache)
    a, b = cache.acquire(), cache.acquire()
    first = step([SequenceInput(a, requests["r0"][:20], [19])]).cpu()
    with pytest.raises(CacheFull):
        step([SequenceInput(a, [1], [0]), SequenceInput(b, list(range(200)), [199])])     # 1 + 4 pages wanted, 3 exist
    assert cache.length(a) == 20 and cache.length(b) == 0
    cache.check_invariants()
    for bad in ([SequenceInput(a, [], [])], [SequenceInput(a, [cfg["vocab_size"]], [0])], [SequenceInput(a, [1], [1])],
                [SequenceInput(a, [1], [0]), SequenceInput(a, [2], [0])], [SequenceInput(77, [1], [0])], []):
        with pytest.raises(StepError):
            step(bad)
    again = step([SequenceInput(b, requests["r0"][:20], [19])]).cpu()       # the other slot, same tokens, same logits
    assert torch.equal(first, again)


def test_slots_given_to_new_sequences_at_the_position_the_old_ones_stopped(session_tmp):
    """A recorded decode step only rewrites what moved when it continues the step before.  New sequences that get
    the same slot numbers, with other pages, and happen to stand one position after the old ones' last step must
    not be taken for a continuation: their page tables have to reach the device."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    cfg_json, norm_std = TINY["A"]
    d = make_model_dir(session_tmp, cfg_json, seed=41, norm_std=norm_std, scale=PEAKED)
    cfg, w = plain_inputs(d)
    model = load_model(d, torch.bfloat16)
    cache = model.new_cache(64 * 8, max_slots=4)
    step = StepFunction(model, cache)
    old = random_prompts(cfg["vocab_size"], [8, 8], seed=1)
    a, b, keep = cache.acquire(), cache.acquire(), cache.acquire()
    step([SequenceInput(a, old[0][:5], []), SequenceInput(b, old[1][:5], [])])
    for t in range(5, 8):                                   # decode steps at positions 5, 6, 7 (the second one is recorded)
        step([SequenceInput(a, [old[0][t]], [0]), SequenceInput(b, [old[1][t]], [0])])
    cache.release(a)
    cache.release(b)
    filler = random_prompts(cfg["vocab_size"], [130], seed=2)[0]
    step([SequenceInput(keep, filler, [])])                 # takes the pages the old sequences gave back
    new_slots = [cache.acquire(), cache.acquire()]
    new = random_prompts(cfg["vocab_size"], [9, 9], seed=3)
    by_slot = dict(zip(sorted(new_slots), new))             # in the order of the old step: slots a, b
    assert sorted(new_slots) == sorted([a, b])
    step([SequenceInput(s, by_slot[s][:8], []) for s in (a, b)])
    out = step([SequenceInput(s, [by_slot[s][8]], [0]) for s in (a, b)])   # position 8 = the old last position + 1
    for i, s in enumerate((a, b)):
        ref = plain_llama.forward(cfg, w, by_slot[s], round_to=torch.bfloat16)[-1]
        assert_close_logits(out[i], ref, torch.bfloat16, f"sequence in slot {s}")
    cache.check_invariants()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_one_step_holds_a_decoded_token_a_chunk_and_a_fresh_prompt(setup, dtype):
    """Three sequences in one step, each at another stage: one goes on by a single token behind 70 cached ones, one
    brings the middle chunk of its prompt (positions 40..99 of 129), one starts.  Then all three go on together by
    one token.  Every place gives the plain implementation's logits for the whole sequence."""
    from conftest import assert_within_plain_noise
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, weights, requests, refs = setup
    if dtype not in refs:
        refs[dtype] = _reference(cfg, weights, requests, dtype)
    model = load_model(d, dtype)
    cache = model.new_cache(64 * 6)
    step = StepFunction(model, cache)
    one, chunk, fresh = requests["r3"], requests["r4"], requests["r0"]            # 100, 129 and 33 tokens
    a, b, c = cache.acquire(), cache.acquire(), cache.acquire()
    step([SequenceInput(a, one[:70], []), SequenceInput(b, chunk[:40], [])])
    out = step([SequenceInput(a, [one[70]], [0]), SequenceInput(b, chunk[40:100], list(range(60))),
                SequenceInput(c, fresh[:20], list(range(20)))]).cpu()
    ref = refs[dtype]
    want = torch.cat([ref["r3"][70:71], ref["r4"][40:100], ref["r0"][:20]])
    assert_close_logits(out, want, dtype, "one token, a middle chunk and a fresh prompt in one step")
    # the few rows of one sequence alone: against the plain implementation's own distance from its float64 run
    exact = {r: plain_llama.forward(cfg, weights, requests[r], dtype=torch.float64) for r in ("r3", "r4", "r0")}
    assert_within_plain_noise(out[0:1], exact["r3"][70:71], ref["r3"][70:71], dtype, "the sequence that goes on by one token")
    out = step([SequenceInput(a, [one[71]], [0]), SequenceInput(b, [chunk[100]], [0]), SequenceInput(c, [fresh[20]], [0])]).cpu()
    for i, (r, p) in enumerate((("r3", 71), ("r4", 100), ("r0", 20))):
        assert_within_plain_noise(out[i:i + 1], exact[r][p:p + 1], ref[r][p:p + 1], dtype, f"then one token each: {r}")
    assert [cache.length(s) for s in (a, b, c)] == [72, 101, 21]
    cache.check_invariants()
