"""Generation through the Python entry point and the command line against the plain
implementation: greedy tokens, sampled tokens for given uniform numbers, batches whose shorter
requests end earlier, long decoding, the first tokens of a sequence."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_llama as P
from conftest import PEAKED, ROOT, TINY, assert_close_logits, make_model_dir, plain_inputs, random_prompts

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")])
def test_greedy_generation_matches_plain(session_tmp, name, dtype):
    from gpullama3.java_b200.engine.api import Engine

    cfg_json, norm_std = TINY[name]
    d = make_model_dir(session_tmp, cfg_json, seed=21, norm_std=norm_std, scale={"embed_tokens": 8.0, "lm_head": 8.0})
    cfg, w = plain_inputs(d)
    lengths = [5, 11, 17] if name == "A" else [1, 7, 30, 64]
    prompts = random_prompts(cfg["vocab_size"], lengths, seed=2)
    engine = Engine.from_folder(d, dtype=dtype, max_tokens=64 * 8, max_batch=4)
    got = engine.generate(prompts, max_new_tokens=8, stop_ids=())
    rt = None if dtype == "float32" else torch.bfloat16
    for p, g in zip(prompts, got):
        if dtype == "float32":
            assert g == P.generate_greedy(cfg, w, p, 8, round_to=rt)
        else:   # a near-tie may flip in bfloat16: every token must be the plain arg-max or within rounding of it
            seq = list(p)
            for tok in g:
                logits = P.forward(cfg, w, seq, round_to=rt)[-1]
                assert float(logits.max() - logits[tok]) <= 4 * 2.0 ** -8 * float(logits.abs().max())
                seq.append(tok)
    assert engine.cache.live_slots() == []
    m = engine.last_metrics
    assert m.prompt_tokens == sum(lengths) and m.generated_tokens == 8 * len(lengths)


def test_stop_tokens_end_sequences_early_and_batches_reuse_slots(session_tmp):
    from gpullama3.java_b200.engine.api import Engine

    cfg_json, norm_std = TINY["A"]
    d = make_model_dir(session_tmp, cfg_json, seed=21, scale={"embed_tokens": 8.0})
    cfg, w = plain_inputs(d)
    prompts = random_prompts(256, [9, 3, 20, 14, 6, 33, 2], seed=4)
    free = [P.generate_greedy(cfg, w, p, 12) for p in prompts]
    stop = {free[0][3], free[4][1]}
    want = [P.generate_greedy(cfg, w, p, 12, stop_ids=stop) for p in prompts]
    assert len({len(x) for x in want}) > 1                           # some end early, some do not
    engine = Engine.from_folder(d, dtype="float32", max_tokens=64 * 3, max_batch=3)   # three batches through 3 slots
    res = engine.generate(prompts, max_new_tokens=12, stop_ids=stop, return_results=True)
    assert [r.tokens for r in res] == want
    assert [r.finish_reason for r in res] == ["stop" if x[-1] in stop else "length" for x in want]
    assert engine.cache.live_slots() == []
    engine.cache.check_invariants()


def test_temperature_sampling_follows_the_uniform_numbers(session_tmp):
    """Tiny B, 16 tokens at temperature 0.8: every sampled token is the inverse-CDF token of the
    plain softmax for the same uniform number, whatever batch the request sits in."""
    from gpullama3.java_b200.engine.api import Engine
    from gpullama3.java_b200.sampling import uniform

    cfg_json, norm_std = TINY["B"]
    d = make_model_dir(session_tmp, cfg_json, seed=22, norm_std=norm_std, scale={"lm_head": 30.0})
    cfg, w = plain_inputs(d)
    prompts = random_prompts(cfg["vocab_size"], [1, 7, 30, 64], seed=5)
    engine = Engine.from_folder(d, dtype="float32", max_tokens=64 * 8, max_batch=4)
    got = engine.generate(prompts, max_new_tokens=16, temperature=0.8, seed=1234, stop_ids=())
    for i, (p, g) in enumerate(zip(prompts, got)):
        seq = list(p)
        for n, tok in enumerate(g):
            probs = P.temperature_softmax(P.forward(cfg, w, seq)[-1], 0.8).double()
            cdf = torch.cumsum(probs, 0)
            u = uniform(1234, i, n)
            lo = float(cdf[tok - 1]) if tok else 0.0
            assert lo - 1e-5 <= u < float(cdf[tok]) + 1e-5, (i, n, tok, u)
            seq.append(tok)
    alone = Engine.from_folder(d, dtype="float32", max_tokens=64 * 2, max_batch=1)
    one = alone.generator.generate([prompts[2]], 16, __import__("gpullama3.java_b200.sampling", fromlist=["SamplingParams"])
                                   .SamplingParams(0.8, 1.0, 1234), (), request_ids=[2])
    assert one[0].tokens == got[2]                                   # same draws alone as in the batch
    # Nucleus sampling through the same loop (the draw recorded with the step): every token is the one the plain
    # sampler takes for the same uniform number (inference/sampler/ToppSampler.java:110-156 of the reference project),
    # or its neighbour in the sorted order when the number falls within rounding of the boundary between them.
    V = cfg["vocab_size"]
    nucleus = engine.generate(prompts, max_new_tokens=8, temperature=0.8, top_p=0.9, seed=5, stop_ids=())
    assert engine.step_fn.last_d2h_bytes > 0                          # the recorded path was taken
    for i, (p, g) in enumerate(zip(prompts, nucleus)):
        assert len(g) == 8
        seq = list(p)
        for n, tok in enumerate(g):
            probs = P.temperature_softmax(P.forward(cfg, w, seq)[-1], 0.8)
            u = uniform(5, i, n)
            want = P.sample_top_p(probs, 0.9, u)
            if tok != want:
                pl = probs.tolist()
                order = sorted(range(V), key=lambda t: (-pl[t], t))
                csum = torch.cumsum(probs[order].double(), 0)
                kept = int((csum <= 0.9).sum()) + 1
                r, j = u * float(csum[kept - 1]), order.index(tok)
                assert j < kept and min(abs(r - float(csum[j])), abs(r - (float(csum[j - 1]) if j else 0.0))) < 1e-5, \
                    (i, n, tok, want, u)
            seq.append(tok)


@pytest.mark.parametrize("sampling", [dict(), dict(temperature=0.7, seed=3), dict(temperature=0.9, top_p=0.8, seed=4)],
                         ids=["greedy", "temperature", "nucleus"])
def test_step_and_draw_recorded_together_give_the_tokens_of_step_then_draw(session_tmp, sampling):
    """Decode steps normally run as one recorded launch that ends with the sampler's kernels and the copy of the
    tokens to the host, launched one step ahead of the tokens the host has read and fed with the tokens of the
    step before on the device; with that switched off the loop waits for each step's tokens, and with the
    recorded draw switched off too it runs the step, then the sampler.  Same tokens all three ways, and the
    recorded path is really taken (it reports the bytes it copied back)."""
    from gpullama3.java_b200.engine.api import Engine

    cfg_json, norm_std = TINY["A"]
    d = make_model_dir(session_tmp, cfg_json, seed=23, norm_std=norm_std, scale={"lm_head": 20.0},
                       max_position_embeddings=1024)        # generation stops at the configuration's context length
    cfg, _ = plain_inputs(d)
    prompts = random_prompts(cfg["vocab_size"], [3, 70, 9, 33], seed=6)
    engine = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 16, max_batch=4)
    together = engine.generate(prompts, max_new_tokens=70, stop_ids=(), **sampling)   # crosses a page boundary
    assert engine.step_fn.last_d2h_bytes > 0
    assert any(key[3] != 0 for key in engine.step_fn._graphs), "no step was fed on the device"
    waiting = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 16, max_batch=4)
    waiting.generator.step_fn.decode_ahead = lambda *a, **k: False
    in_turn = waiting.generate(prompts, max_new_tokens=70, stop_ids=(), **sampling)
    assert waiting.step_fn.last_d2h_bytes > 0 and all(key[3] == 0 for key in waiting.step_fn._graphs)
    apart_engine = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 16, max_batch=4)
    apart_engine.generator.step_fn.decode_ahead = lambda *a, **k: False
    apart_engine.generator.step_fn.decode_and_sample = lambda *a, **k: None
    apart = apart_engine.generate(prompts, max_new_tokens=70, stop_ids=(), **sampling)
    assert apart_engine.step_fn.last_d2h_bytes == 0
    assert together == in_turn == apart


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_long_decoding_and_first_tokens(session_tmp, dtype):
    """One token a step from the very first token on, for 330 positions (five page boundaries), and
    the first three positions of a sequence on their own."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    cfg_json, norm_std = TINY["B"]
    d = make_model_dir(session_tmp, cfg_json, seed=23, norm_std=norm_std, scale=PEAKED)
    cfg, w = plain_inputs(d)
    toks = random_prompts(cfg["vocab_size"], [330], seed=6)[0]
    ref = P.forward(cfg, w, toks, round_to=None if dtype == torch.float32 else torch.bfloat16)
    model = load_model(d, dtype)
    cache = model.new_cache(64 * 6)
    step = StepFunction(model, cache)
    slot = cache.acquire()
    rows = [step([SequenceInput(slot, [t], [0])])[0] for t in toks]
    assert_close_logits(torch.stack(rows), ref, dtype, "token by token from position 0")
    assert_close_logits(torch.stack(rows[:3]), ref[:3], dtype, "first tokens")
    cache.release(slot)
    for n in (1, 2, 3):
        slot = cache.acquire()
        out = step([SequenceInput(slot, toks[:n], list(range(n)))])
        assert_close_logits(out, ref[:n], dtype, f"first {n} tokens in one step")
        cache.release(slot)


def test_command_line(session_tmp, tmp_path):
    cfg_json, _ = TINY["A"]
    d = make_model_dir(session_tmp, cfg_json, seed=21, scale={"embed_tokens": 8.0})
    cfg, w = plain_inputs(d)
    env = dict(os.environ, PYTHON=sys.executable)
    cmd = [str(ROOT / "bin" / "llama-b200"), "--model", str(d), "--dtype", "float32", "--temperature", "0",
           "-n", "6", "--stream", "false", "--prompt", "3 1 4 1 5", "--prompt", "9,2,6", "--stop", "300"]
    p = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.strip().splitlines() if l.strip()]
    assert [list(map(int, l.split())) for l in lines] == [P.generate_greedy(cfg, w, [3, 1, 4, 1, 5], 6),
                                                          P.generate_greedy(cfg, w, [9, 2, 6], 6)]
    assert "achieved tok/s" in p.stderr
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    p = subprocess.run([str(ROOT / "bin" / "llama-b200"), "--config", str(tmp_path / "config.json"), "--random-weights", "3",
                        "--prompt", "1 2 3", "-n", "4", "--seed", "1"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0 and len(p.stdout.split()) == 4, p.stderr[-2000:]
    # a position cap, the kernel table and the timing line
    p = subprocess.run(cmd[:-2] + ["--max-len", "8", "--profile", "--bench"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [list(map(int, l.split())) for l in p.stdout.strip().splitlines() if l.strip()]
    assert lines == [P.generate_greedy(cfg, w, [3, 1, 4, 1, 5], 3), P.generate_greedy(cfg, w, [9, 2, 6], 5)]   # 8 positions each
    assert "b200_gemm_generic" in p.stderr and "b200_attention_paged" in p.stderr and "mean us" in p.stderr
    timing = [json.loads(l) for l in p.stderr.splitlines() if l.startswith("{")]
    assert timing and timing[0]["prompt_tokens"] == 8 and timing[0]["generated_tokens"] == 8 and timing[0]["decode_tokens_per_s"] > 0


def test_steps_launched_ahead_keep_their_tokens_when_the_page_tables_grow(session_tmp):
    """330 new tokens on prompts of 3, 200 and 40: the page tables of the recorded steps double twice on the way
    (4, 8, 16 pages wide), so device-fed steps are recorded anew in mid-flight, each while the step before it
    runs.  Same tokens as the loop that waits for every step."""
    from gpullama3.java_b200.engine.api import Engine

    cfg_json, norm_std = TINY["A"]
    d = make_model_dir(session_tmp, cfg_json, seed=23, norm_std=norm_std, scale={"lm_head": 20.0},
                       max_position_embeddings=1024)
    prompts = random_prompts(cfg_json["vocab_size"], [3, 200, 40], seed=6)
    ahead = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 32, max_batch=4)
    got = ahead.generate(prompts, max_new_tokens=330, stop_ids=(), temperature=0.7, seed=3)
    fed_widths = sorted(key[1] for key in ahead.step_fn._graphs if key[3] != 0)
    assert fed_widths == [(4,), (4,), (8,), (8,), (16,), (16,)]
    waiting = Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 32, max_batch=4)
    waiting.generator.step_fn.decode_ahead = lambda *a, **k: False
    assert got == waiting.generate(prompts, max_new_tokens=330, stop_ids=(), temperature=0.7, seed=3)
    assert [len(t) for t in got] == [330, 330, 330]
    ahead.cache.check_invariants()
