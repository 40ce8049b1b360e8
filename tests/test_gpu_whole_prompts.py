"""Each request alone and whole: the engine's logits at every position against the plain
implementation, for both tiny configurations, both precisions and both rotary pairings."""
import pytest
import torch

import plain_llama
from conftest import TINY, assert_close_logits, make_model_dir, plain_inputs, random_prompts

pytestmark = pytest.mark.gpu


def engine_logits_whole(model_dir, dtype, prompts, max_tokens=1024):
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    model = load_model(model_dir, dtype)
    cache = model.new_cache(max_tokens)
    step = StepFunction(model, cache)
    outs = []
    for p in prompts:
        slot = cache.acquire()
        outs.append(step([SequenceInput(slot, list(p), list(range(len(p))))]).cpu())
        cache.release(slot)
    cache.check_invariants()
    return outs


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
def test_whole_prompt_matches_plain(session_tmp, name, dtype, pairing):
    cfg_json, norm_std = TINY[name]
    d = make_model_dir(session_tmp, cfg_json, seed=1, norm_std=norm_std, rope_pairing=pairing)
    cfg, weights = plain_inputs(d)
    g = torch.Generator().manual_seed(5)
    lengths = [1, 7, 30, 64, 65, 130]
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]
    got = engine_logits_whole(d, dtype, prompts)
    for p, out in zip(prompts, got):
        ref = plain_llama.forward(cfg, weights, p, round_to=None if dtype == torch.float32 else torch.bfloat16)
        assert_close_logits(out, ref, dtype, f"tiny {name} {pairing} len {len(p)}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_passes_take_their_tensors_from_one_block_of_memory(session_tmp, dtype):
    """The second prompt pass asks nothing of the allocator for its intermediate tensors (the first sized the
    block), and the logits are the bits of a pass that takes every tensor from the allocator."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    cfg_json, norm_std = TINY["B"]
    d = make_model_dir(session_tmp, cfg_json, seed=1, norm_std=norm_std)
    model = load_model(d, dtype)
    cache = model.new_cache(64 * 8)
    step = StepFunction(model, cache)
    prompts = random_prompts(cfg_json["vocab_size"], [70, 9, 33], seed=3)

    def run():
        slots = [cache.acquire() for _ in prompts]
        out = step([SequenceInput(s, p, [0, len(p) - 1]) for s, p in zip(slots, prompts)]).clone()
        for s in slots:
            cache.release(s)
        return out

    first = run()
    assert step.workspace.overflowed > 0 and step.workspace.capacity == 0     # nothing was kept yet
    second = run()
    asked = step.workspace.overflowed
    third = run()
    assert step.workspace.capacity > 0 and step.workspace.overflowed == asked  # the third pass fitted entirely
    step.workspace = None
    plain = run()
    assert torch.equal(first, plain) and torch.equal(second, plain) and torch.equal(third, plain)
