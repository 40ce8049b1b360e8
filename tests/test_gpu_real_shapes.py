"""The layer sizes of the real models (Llama-3.2-3B and Llama-3.1-8B: head size 128, 24 or 32 heads over 8 kv
heads, widths 3072/4096, feed-forward 8192/14336) with two layers and a short vocabulary: prompts in one step and
then decoded tokens, in both precisions, against the plain implementation.  These sizes take the tensor-core
kernels' other template instances (head_dim 128, groups of 3 and 4, K = 14336, prefill tiles with ragged edges)."""
import pytest
import torch

import plain_llama as P
from conftest import make_model_dir, plain_inputs, random_prompts

pytestmark = pytest.mark.gpu

SHAPES = {
    "3B": dict(hidden_size=3072, num_attention_heads=24, num_key_value_heads=8, head_dim=128, intermediate_size=8192,
               rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192}, tie_word_embeddings=True),
    "8B": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336,
               rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192}, tie_word_embeddings=False),
}


@pytest.mark.parametrize("name", ["3B", "8B"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_layers_of_real_size(session_tmp, name, dtype):
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    cfg_json = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, vocab_size=1000, rope_theta=500000.0,
                    rms_norm_eps=1e-5, max_position_embeddings=8192, **SHAPES[name])
    d = make_model_dir(session_tmp, cfg_json, seed=31)   # N(0, 0.02): at these widths the scores already spread over a few units
    cfg, w = plain_inputs(d)
    lengths = [150, 37, 70]           # 257 tokens in the prompt step: more than two prefill tiles, a ragged edge
    prompts = random_prompts(1000, lengths, seed=8)
    tail = 6
    rt = None if dtype == torch.float32 else torch.bfloat16
    refs = [P.forward(cfg, w, p, round_to=rt) for p in prompts]
    # Sums of 8192 and 14336 terms: round-off itself is no longer small against the tiny models' tolerances, so
    # the yardstick here is the plain implementation's own error (float32, or rounded to bfloat16 at the places
    # where the engine rounds) against its float64 run: on the same rows the engine may be twice (bfloat16) or
    # four times (float32, whose noise is tiny) that far from the float64 logits, not more.
    exact = [P.forward(cfg, w, p, dtype=torch.float64) for p in prompts]
    scale = max(float(e.abs().max()) for e in exact)
    factor = 4.0 if dtype == torch.float32 else 2.0

    def check(got, i, rows, what):
        g, e, r = got.cpu().double(), exact[i][rows].double(), refs[i][rows].double()
        assert torch.isfinite(g).all(), what
        err, noise = float((g - e).abs().max()), float((r - e).abs().max())
        assert err <= factor * noise + 2e-5 * scale, f"{what}: max err {err:.3e}, plain noise {noise:.3e}, scale {scale:.3e}"
        err_m, noise_m = float((g - e).abs().mean()), float((r - e).abs().mean())
        assert err_m <= factor * noise_m + 2e-6 * scale, f"{what}: mean err {err_m:.3e}, plain noise {noise_m:.3e}"

    model = load_model(d, dtype)
    cache = model.new_cache(64 * 8)
    step = StepFunction(model, cache)
    slots = [cache.acquire() for _ in prompts]
    heads = [n - tail for n in lengths]
    out = step([SequenceInput(s, p[:h], list(range(h))) for s, p, h in zip(slots, prompts, heads)])
    off = 0
    for i, h in enumerate(heads):
        check(out[off:off + h], i, slice(0, h), f"{name} prompt {i}")
        off += h
    for t in range(tail):
        out = step([SequenceInput(s, [p[h + t]], [0]) for s, p, h in zip(slots, prompts, heads)])
        for i, h in enumerate(heads):
            check(out[i:i + 1], i, slice(h + t, h + t + 1), f"{name} decoded token {t} of {i}")
    for s in slots:
        cache.release(s)


@pytest.mark.parametrize("name", ["1B", "3B"])
def test_long_prompts_of_real_size(session_tmp, name):
    """Prompts of 700, 260 and 130 tokens with 32 (24) heads make more attention work than there are SMs: the prompt
    step takes the kernel that handles query tiles in pairs (head sizes 64 and 128), the decode steps after it cut
    the 700 keys into spans.  One layer, bfloat16, the yardstick of the test above."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model
    from gpullama3.java_b200.kernels import ops

    shape = SHAPES["3B"] if name == "3B" else dict(
        hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192,
        rope_scaling=SHAPES["3B"]["rope_scaling"], tie_word_embeddings=True)
    cfg_json = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=1, vocab_size=1000, rope_theta=500000.0,
                    rms_norm_eps=1e-5, max_position_embeddings=8192, **shape)
    d = make_model_dir(session_tmp, cfg_json, seed=33)
    cfg, w = plain_inputs(d)
    lengths = [700, 260, 130]
    assert -(-max(lengths) // 256) * cfg["num_attention_heads"] * len(lengths) >= 148
    prompts = random_prompts(1000, lengths, seed=9)
    tail = 3
    refs = [P.forward(cfg, w, p, round_to=torch.bfloat16) for p in prompts]
    exact = [P.forward(cfg, w, p, dtype=torch.float64) for p in prompts]
    scale = max(float(e.abs().max()) for e in exact)

    def check(got, i, rows, what):
        g, e, r = got.cpu().double(), exact[i][rows].double(), refs[i][rows].double()
        assert torch.isfinite(g).all(), what
        err, noise = float((g - e).abs().max()), float((r - e).abs().max())
        assert err <= 2.0 * noise + 2e-5 * scale, f"{what}: max err {err:.3e}, plain noise {noise:.3e}, scale {scale:.3e}"
        err_m, noise_m = float((g - e).abs().mean()), float((r - e).abs().mean())
        assert err_m <= 2.0 * noise_m + 2e-6 * scale, f"{what}: mean err {err_m:.3e}, plain noise {noise_m:.3e}"

    model = load_model(d, torch.bfloat16)
    cache = model.new_cache(64 * 20)
    step = StepFunction(model, cache)
    slots = [cache.acquire() for _ in prompts]
    heads = [n - tail for n in lengths]
    wanted = [list(range(0, h, 37)) + [h - 1] for h in heads]      # rows spread over every tile, and the last one
    out = step([SequenceInput(s, p[:h], rows) for s, p, h, rows in zip(slots, prompts, heads, wanted)])
    assert ops.attention_prefill_tc_status() == 0
    off = 0
    for i, rows in enumerate(wanted):
        check(out[off:off + len(rows)], i, rows, f"{name} prompt {i}")
        off += len(rows)
    for t in range(tail):
        out = step([SequenceInput(s, [p[h + t]], [0]) for s, p, h in zip(slots, prompts, heads)])
        for i, h in enumerate(heads):
            check(out[i:i + 1], i, slice(h + t, h + t + 1), f"{name} decoded token {t} of {i}")
    for s in slots:
        cache.release(s)


# --------------------------------------------------------------------------- the replay cuts at these sizes
SIZES = {
    "1B": dict(hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192,
               rope_scaling=SHAPES["3B"]["rope_scaling"], tie_word_embeddings=True),
    "3B": SHAPES["3B"],
    "8B": SHAPES["8B"],
}
CUT_LENGTHS = [1600, 520, 300, 180, 100, 45]


@pytest.fixture(scope="module", params=["1B", "3B", "8B"])
def sized(request, session_tmp):
    cfg_json = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, vocab_size=1000, rope_theta=500000.0,
                    rms_norm_eps=1e-5, max_position_embeddings=8192, **SIZES[request.param])
    d = make_model_dir(session_tmp, cfg_json, seed=35)
    cfg, w = plain_inputs(d)
    w = {k: t.cuda() for k, t in w.items()}          # the plain implementation's arithmetic, evaluated on the GPU
    requests = {f"r{i}": p for i, p in enumerate(random_prompts(1000, CUT_LENGTHS, seed=12))}
    exact = {r: P.forward(cfg, w, t, dtype=torch.float64, device="cuda") for r, t in requests.items()}
    return request.param, d, cfg, w, requests, exact, {}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("cut", ["whole", "tail32", "batches3"])
def test_replay_cuts_at_real_layer_sizes(sized, tmp_path, dtype, cut):
    """The three ways of cutting the same requests (each alone and whole; the last 32 tokens one by one; batches of
    three with unequal prompts whose shorter requests end earlier, the second batch in the pages the first gave
    back) with two layers of the 1B, 3B and 8B sizes.  A request of 1,600 tokens alone is more attention work than
    there are SMs (the kernel that takes query tiles in pairs), prompts of a few hundred tokens take the product
    that cuts K into spans, and decoding behind 1,400 cached tokens cuts the keys into spans."""
    from gpullama3.java_b200.engine.trace import load_model
    from gpullama3.java_b200.kernels import ops
    from replay_helpers import max_live_tokens, read_rows, run_in_process, trace_batches, trace_tail_one_by_one, trace_whole

    name, d, cfg, w, requests, exact, refs = sized
    rt = None if dtype == torch.float32 else torch.bfloat16
    if dtype not in refs:
        refs[dtype] = {r: P.forward(cfg, w, t, round_to=rt, device="cuda") for r, t in requests.items()}
    if cut == "whole":
        steps, rows = trace_whole(requests)
    elif cut == "tail32":
        steps, rows = trace_tail_one_by_one(requests, 32)
    else:
        steps, rows = trace_batches(requests, 3, prompt_fraction=0.9)
    model = load_model(d, dtype)
    before = ops.launches_by_kernel()
    run_in_process(model, steps, tmp_path, max_live_tokens(steps))
    after = ops.launches_by_kernel()
    ran = {k for k in after if after[k] != before.get(k, 0)}
    if dtype == torch.bfloat16:
        assert ops.gemm_tcgen05_status() == 0 and ops.attention_prefill_tc_status() == 0
        assert not ({"gemm_generic", "attention_paged", "attention_prefill"} & ran), ran
        assert {"gemm_tcgen05", "attention_prefill_tc"} <= ran, ran
        if cut != "whole":
            assert {"attention_decode_rope", "gemm_decode_linked"} <= ran, ran
        else:   # the long prompts rotate and fill the cache in the projection's epilogue, the short ones in a kernel of its own
            assert {"gemm_tcgen05_qkv_rope", "rope_angles", "rope_cache_write"} <= ran, ran
        hidden, inner = cfg["hidden_size"], cfg["intermediate_size"]
        rows_of_passes = [sum(len(e["tokens"]) for e in s["entries"]) for s in steps]
        if cut == "tail32":     # prompts of 13 to 1,568 tokens alone: some of them are few tiles with a long K
            assert any(m > 128 and ops.gemm_tcgen05_k_spans(m, hidden, inner) > 1 for m in rows_of_passes), rows_of_passes
    got = read_rows(tmp_path, rows, 1000)
    factor = 4.0 if dtype == torch.float32 else 2.0
    by_req: dict = {}
    for (rid, pos), row in got.items():
        by_req.setdefault(rid, []).append((pos, row))
    for rid, items in by_req.items():
        items.sort()
        at = [p for p, _ in items]
        g, e, r = torch.stack([x for _, x in items]).double(), exact[rid][at].double(), refs[dtype][rid][at].double()
        scale = float(exact[rid].abs().max())
        assert torch.isfinite(g).all(), f"{name} {cut} {rid}"
        err, noise = float((g - e).abs().max()), float((r - e).abs().max())
        assert err <= factor * noise + 2e-5 * scale, f"{name} {cut} {rid}: max err {err:.3e}, plain noise {noise:.3e}, scale {scale:.3e}"
        err_m, noise_m = float((g - e).abs().mean()), float((r - e).abs().mean())
        assert err_m <= factor * noise_m + 2e-6 * scale, f"{name} {cut} {rid}: mean err {err_m:.3e}, plain noise {noise_m:.3e}"
