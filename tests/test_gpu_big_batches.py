"""Many sequences decoding together (17, 64, 128), through the model, against the plain implementation.

Up to 16 sequences a decode step's products are the weight-streaming kernel with the norms folded into them; from 17
on they are the few-token tensor-core product with norm kernels of their own, and a batch of long sequences that
fills the GPU starts its attention late.  The tiny models take these paths with every head and group count of the two
configurations; a two-layer model with the layer sizes of Llama-3.2-1B takes the tensor-core kernels themselves, and
the test asserts that they ran."""
import pytest
import torch

import plain_llama as P
from conftest import PEAKED, TINY, assert_close_logits, make_model_dir, plain_inputs, random_prompts
from replay_helpers import max_live_tokens, read_rows, run_in_process, trace_batches

pytestmark = pytest.mark.gpu


def _requests(vocab, n, lengths, seed):
    prompts = random_prompts(vocab, [lengths[i % len(lengths)] for i in range(n)], seed=seed)
    return {f"r{i}": p for i, p in enumerate(prompts)}


@pytest.fixture(scope="module", params=["A", "B"])
def tiny(request, session_tmp):
    cfg_json, norm_std = TINY[request.param]
    d = make_model_dir(session_tmp, cfg_json, seed=17, norm_std=norm_std, scale=PEAKED)
    cfg, weights = plain_inputs(d)
    return d, cfg, weights, {}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("n", [17, 64, 128])
def test_many_sequences_decode_together(tiny, tmp_path, dtype, n):
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, weights, refs = tiny
    # prompts of 6 to 39 tokens, then 4 to 26 tokens one by one: the batch shrinks from n in five stages
    requests = _requests(cfg["vocab_size"], n, [10, 65, 33, 20, 47], seed=n)
    steps, rows = trace_batches(requests, n, prompt_fraction=0.6)
    assert max(len(s["entries"]) for s in steps[1:]) == n
    model = load_model(d, dtype)
    run_in_process(model, steps, tmp_path, max_live_tokens(steps))
    got = read_rows(tmp_path, rows, cfg["vocab_size"])
    rt = None if dtype == torch.float32 else torch.bfloat16
    by_req: dict = {}
    for (rid, pos), row in got.items():
        by_req.setdefault(rid, []).append((pos, row))
    for rid, items in by_req.items():
        key = (rid, n, dtype)
        if key not in refs:
            refs[key] = P.forward(cfg, weights, requests[rid], round_to=rt)
        items.sort()
        assert_close_logits(torch.stack([r for _, r in items]), refs[key][[p for p, _ in items]], dtype,
                            f"{n} sequences, request {rid}")


SIZE_1B = dict(architectures=["LlamaForCausalLM"], num_hidden_layers=2, vocab_size=1000, rope_theta=500000.0,
               rms_norm_eps=1e-5, max_position_embeddings=8192, hidden_size=2048, num_attention_heads=32,
               num_key_value_heads=8, head_dim=64, intermediate_size=8192, tie_word_embeddings=True,
               rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192})


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("n", [17, 64, 128])
def test_many_sequences_at_the_layer_sizes_of_the_1b_model(session_tmp, tmp_path, dtype, n):
    """One of the sequences is 1,700 tokens long (1,530 of them in the prompt step): with 64 sequences or more
    its page table makes the decode attention a grid that fills the GPU with long spans, which is launched without
    an early start."""
    from gpullama3.java_b200.engine.trace import load_model
    from gpullama3.java_b200.kernels import ops

    d = make_model_dir(session_tmp, SIZE_1B, seed=37)
    cfg, w = plain_inputs(d)
    requests = _requests(1000, n - 1, [30, 75, 12, 140], seed=n + 1)
    requests["long"] = random_prompts(1000, [1700], seed=5)[0]
    steps, rows = trace_batches(requests, n, prompt_fraction=0.9)
    model = load_model(d, dtype)
    before = ops.launches_by_kernel()
    run_in_process(model, steps, tmp_path, max_live_tokens(steps))
    after = ops.launches_by_kernel()
    ran = {k: after[k] - before.get(k, 0) for k in after if after[k] != before.get(k, 0)}
    if dtype == torch.bfloat16:
        assert ran.get("gemm_skinny", 0) > 0, ran            # 17 to 128 rows: the few-token tensor-core product
        assert ops.gemm_skinny_status() == 0
        if n >= 64:
            assert ran.get("attention_decode_rope:late", 0) > 0, ran
        assert "gemm_generic" not in ran and "attention_paged" not in ran, ran
    else:
        assert set(ran) <= {"embed_gather", "rmsnorm", "rope_cache_write", "attention_paged", "gemm_generic"}, ran
    got = read_rows(tmp_path, rows, 1000)
    w = {k: t.cuda() for k, t in w.items()}                  # the plain implementation's arithmetic, evaluated on the GPU
    rt = None if dtype == torch.float32 else torch.bfloat16
    factor = 4.0 if dtype == torch.float32 else 2.0
    by_req: dict = {}
    for (rid, pos), row in got.items():
        by_req.setdefault(rid, []).append((pos, row))
    for rid, items in by_req.items():
        items.sort()
        at = [p for p, _ in items]
        g = torch.stack([r for _, r in items]).double()
        exact = P.forward(cfg, w, requests[rid], dtype=torch.float64, device="cuda")[at].double()
        ref = P.forward(cfg, w, requests[rid], round_to=rt, device="cuda")[at].double()
        scale = float(exact.abs().max())
        assert torch.isfinite(g).all()
        err, noise = float((g - exact).abs().max()), float((ref - exact).abs().max())
        assert err <= factor * noise + 2e-5 * scale, f"{n} sequences, request {rid}: max err {err:.3e}, plain noise {noise:.3e}"
        err_m, noise_m = float((g - exact).abs().mean()), float((ref - exact).abs().mean())
        assert err_m <= factor * noise_m + 2e-6 * scale, f"{n} sequences, request {rid}: mean err {err_m:.3e}, plain noise {noise_m:.3e}"
