"""Shared fixtures: the two tiny Llama 3 configurations, random model folders, tolerances."""
from __future__ import annotations

import json
import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# The two tiny configurations differ in every size and option: layers, width, heads and groups
# (4/2 against 3/1), head size, feed-forward width, vocabulary, rope base and scaling, eps, tying,
# norm weights (ones against 1 + N(0, 0.1)).
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 192, "vocab_size": 256, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 128,
    "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256, "vocab_size": 384, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256, "eos_token_id": [3, 5],
}
TINY = {"A": (TINY_A, 0.0), "B": (TINY_B, 0.1)}  # name -> (config.json, std of the norm weights around 1)


def make_model_dir(tmp_path: Path, config_json: dict, seed: int = 0, norm_std: float = 0.0,
                   dtype=torch.bfloat16, norm_dtype=None, scale: dict | None = None, **overrides) -> Path:
    """Write a random model folder for ``config_json`` (with overrides) and return its path.
    ``scale`` maps a substring of checkpoint names to a factor (``{"q_proj": 8.0}``): it makes the
    attention peaked so that a single wrong key or cache slot changes the logits visibly."""
    from gpullama3.java_b200.config import config_from_dict
    from gpullama3.java_b200.weights import random_checkpoint, write_safetensors

    d = dict(config_json)
    d.update(overrides)
    cfg = config_from_dict(d)
    tag = json.dumps([d, seed, norm_std, str(dtype), str(norm_dtype), scale], sort_keys=True)
    out = tmp_path / f"model_{abs(hash(tag)) % 10**10}"
    if (out / "model.safetensors").is_file():
        return out
    out.mkdir(parents=True, exist_ok=True)
    # the device makes the same bits as the CPU (tests/test_gpu_random_weights.py), only much faster at real layer sizes
    where = "cuda" if torch.cuda.is_available() else "cpu"
    tensors = {n: t.cpu() for n, t in random_checkpoint(cfg, seed, dtype=dtype, norm_std=norm_std, norm_dtype=norm_dtype,
                                                        device=where)}
    for key, factor in (scale or {}).items():
        for name in tensors:
            if key in name:
                tensors[name] = (tensors[name].to(torch.float32) * factor).to(tensors[name].dtype)
    (out / "config.json").write_text(json.dumps(cfg.to_dict(), indent=2))
    write_safetensors(out / "model.safetensors", tensors)
    return out


def plain_inputs(model_dir: Path):
    """config.json as a dict and the weights as float32 tensors by checkpoint name, read with the
    safetensors package (not with the product's reader)."""
    from safetensors.torch import load_file

    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    weights = {k: v.to(torch.float32) for k, v in load_file(str(Path(model_dir) / "model.safetensors")).items()}
    return cfg, weights


# Tolerances, fixed once.  float32: accumulation-order noise only.  bfloat16: the plain
# implementation rounds activations to bfloat16 at the same places as the engine, what remains are
# roundings that fall on the other side of a tie (2^-8 relative on single values).
BF16_EPS = 2.0 ** -8


def assert_close_logits(got: torch.Tensor, ref: torch.Tensor, dtype, what: str = "") -> None:
    got = got.detach().to("cpu", torch.float32)
    ref = ref.detach().to("cpu", torch.float32)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = float(ref.abs().max()) + 1e-30
    err = (got - ref).abs()
    if dtype == torch.float32:
        assert float(err.max()) <= 2e-5 * scale, f"{what}: max err {float(err.max()):.3e} vs scale {scale:.3e}"
    else:
        assert float(err.max()) <= 4 * BF16_EPS * scale, f"{what}: max err {float(err.max()):.3e} vs scale {scale:.3e}"
        assert float(err.mean()) <= 0.5 * BF16_EPS * scale, f"{what}: mean err {float(err.mean()):.3e} vs scale {scale:.3e}"


def assert_within_plain_noise(got, exact, ref, dtype, what: str = "") -> None:
    """For a handful of rows, where the mean of ``assert_close_logits`` has too few numbers under it: the yardstick
    is the plain implementation's own distance (float32, or rounded to bfloat16 where the engine rounds) from its
    float64 run on the same rows.  The engine may be twice (bfloat16) or four times (float32, whose noise is tiny) as
    far from the float64 logits, not more."""
    g, e, r = (t.detach().to("cpu", torch.float64) for t in (got, exact, ref))
    assert g.shape == e.shape == r.shape, f"{what}: shapes {tuple(g.shape)}, {tuple(e.shape)}, {tuple(r.shape)}"
    assert torch.isfinite(g).all(), f"{what}: non-finite logits"
    factor = 4.0 if dtype == torch.float32 else 2.0
    scale = float(e.abs().max()) + 1e-30
    err, noise = float((g - e).abs().max()), float((r - e).abs().max())
    assert err <= factor * noise + 2e-5 * scale, f"{what}: max err {err:.3e}, plain noise {noise:.3e}, scale {scale:.3e}"
    err_m, noise_m = float((g - e).abs().mean()), float((r - e).abs().mean())
    assert err_m <= factor * noise_m + 2e-6 * scale, f"{what}: mean err {err_m:.3e}, plain noise {noise_m:.3e}"


@pytest.fixture(scope="session")
def session_tmp(tmp_path_factory):
    return tmp_path_factory.mktemp("models")


PEAKED = {"q_proj": 8.0, "k_proj": 8.0}  # attention scores of a few units: single keys matter


def random_prompts(vocab: int, lengths, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
