"""The plain implementation checked against itself and against hand-computed values (no GPU)."""
import math

import pytest
import torch

import plain_llama as P
from conftest import TINY, make_model_dir, plain_inputs


def test_rmsnorm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    r = 1.0 / math.sqrt((9 + 16) / 2 + 1e-5)
    assert torch.allclose(P.rmsnorm(x, w, 1e-5), torch.tensor([[2 * 3 * r, 0.5 * 4 * r]]), atol=1e-6)


def test_rope_scaling_hits_all_three_branches_in_tiny_b():
    cfg = TINY["B"][0]
    plain = P.rope_inverse_frequencies(32, 5e5, None)
    scaled = P.rope_inverse_frequencies(32, 5e5, cfg["rope_scaling"])
    ratio = (scaled / plain).tolist()
    assert any(abs(r - 1.0) < 1e-6 for r in ratio)            # short wavelengths kept
    assert any(abs(r - 1 / 8) < 1e-6 for r in ratio)          # long wavelengths slowed by the factor
    assert any(1 / 8 + 1e-3 < r < 1 - 1e-3 for r in ratio)    # the blended band
    assert abs(float(plain[1]) - 5e5 ** (-2 / 32)) < 1e-7


def test_rope_pairings_are_the_same_rotation_on_permuted_dims():
    T, H, D = 5, 2, 8
    x = torch.randn(T, H, D)
    cos, sin = P.rope_tables(torch.arange(T), P.rope_inverse_frequencies(D, 1e4, None), torch.float32)
    perm = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7])             # interleaved layout -> half layout
    a = P.apply_rope(x, cos, sin, "interleaved")[..., perm]
    b = P.apply_rope(x[..., perm], cos, sin, "half")
    assert torch.allclose(a, b, atol=1e-6)
    assert torch.allclose(P.apply_rope(x, cos, sin, "half")[0], x[0])   # position 0 rotates nothing


def test_attention_by_hand_and_window():
    q = torch.tensor([[[1.0, 0.0]], [[1.0, 0.0]]])           # T=2, H=1, D=2
    k = torch.tensor([[[1.0, 0.0]], [[3.0, 0.0]]])
    v = torch.tensor([[[1.0, 2.0]], [[5.0, 6.0]]])
    out = P.causal_attention(q, k, v)
    assert torch.allclose(out[0, 0], v[0, 0])                 # the first token sees only itself
    s = torch.tensor([1.0, 3.0]) / math.sqrt(2)
    p = torch.softmax(s, 0)
    assert torch.allclose(out[1, 0], p[0] * v[0, 0] + p[1] * v[1, 0], atol=1e-6)
    assert torch.allclose(P.causal_attention(q, k, v, window=1)[1, 0], v[1, 0])


def test_grouped_heads_share_their_kv_head():
    T, D = 4, 4
    q = torch.randn(T, 4, D)
    k, v = torch.randn(T, 2, D), torch.randn(T, 2, D)
    out = P.causal_attention(q, k, v)
    solo = P.causal_attention(q[:, 2:3], k[:, 1:2], v[:, 1:2])   # head 2 reads kv head 2 // 2 = 1
    assert torch.allclose(out[:, 2], solo[:, 0], atol=1e-6)


@pytest.mark.parametrize("name", ["A", "B"])
def test_logits_of_a_prefix_do_not_depend_on_what_follows(tmp_path, name):
    cfg_json, norm_std = TINY[name]
    cfg, w = plain_inputs(make_model_dir(tmp_path, cfg_json, seed=4, norm_std=norm_std))
    toks = torch.randint(0, cfg["vocab_size"], (40,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = P.forward(cfg, w, toks)
    assert whole.shape == (40, cfg["vocab_size"])
    for n in (1, 13, 33):
        assert torch.allclose(P.forward(cfg, w, toks[:n]), whole[:n], atol=2e-6)
    w64 = P.forward(cfg, w, toks, dtype=torch.float64)
    assert float((whole - w64).abs().max()) < 1e-5 * float(w64.abs().max()) + 1e-7


def test_tied_and_untied_heads(tmp_path):
    cfg, w = plain_inputs(make_model_dir(tmp_path, TINY["A"][0], seed=4))
    assert "lm_head.weight" not in w
    a = P.forward(cfg, w, [1, 2, 3])
    w2 = dict(w, **{"lm_head.weight": w["model.embed_tokens.weight"] * 2})
    assert torch.allclose(P.forward(cfg, w2, [1, 2, 3]), 2 * a, atol=1e-6)


def test_samplers():
    logits = torch.tensor([0.5, 2.0, 2.0, -1.0])
    assert P.argmax_first(logits) == 1                        # first maximum wins
    p = P.temperature_softmax(logits, 0.5)
    assert abs(float(p.sum()) - 1) < 1e-6 and torch.allclose(p, torch.softmax(logits / 0.5, 0), atol=1e-7)
    cdf = torch.cumsum(p, 0)
    assert P.sample_categorical(p, 0.0) == 0
    assert P.sample_categorical(p, float(cdf[0]) + 1e-4) == 1
    assert P.sample_categorical(p, float(cdf[1]) + 1e-4) == 2
    assert P.sample_categorical(p, 0.99999999) == 3
    probs = torch.tensor([0.05, 0.4, 0.3, 0.2, 0.05])
    # nucleus 0.6: 0.4 + 0.3 = 0.7 > 0.6 -> tokens {1, 2}; r = u * 0.7
    assert P.sample_top_p(probs, 0.6, 0.0) == 1
    assert P.sample_top_p(probs, 0.6, 0.5) == 1               # r = 0.35 < 0.4
    assert P.sample_top_p(probs, 0.6, 0.6) == 2               # r = 0.42 >= 0.4
    assert P.sample_top_p(probs, 0.6, 0.999) == 2
    assert {P.sample_top_p(probs, 0.95, u / 20) for u in range(20)} == {1, 2, 3, 0}   # ties by index: 0 before 4


def test_greedy_generation_keeps_the_stop_token(tmp_path):
    cfg, w = plain_inputs(make_model_dir(tmp_path, TINY["A"][0], seed=4))
    free = P.generate_greedy(cfg, w, [3, 1, 4], 6)
    assert len(free) == 6
    stopped = P.generate_greedy(cfg, w, [3, 1, 4], 6, stop_ids={free[2]})
    assert stopped == free[:free.index(free[2]) + 1]
