"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B
from gpullama3.java_b200.config import (ConfigError, LlamaConfig, config_from_dict, load_config, register_architecture,
                                        registered_architectures, unregister_architecture)


def test_reads_every_key_of_tiny_b():
    c = config_from_dict(TINY_B)
    assert isinstance(c, LlamaConfig)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 96, 3, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size, c.max_position_embeddings) == (32, 256, 384, 256)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0 and not c.tie_word_embeddings
    s = c.rope_scaling
    assert (s.rope_type, s.factor, s.low_freq_factor, s.high_freq_factor, s.original_max_position_embeddings) == \
        ("llama3", 8.0, 1.0, 4.0, 32)
    assert c.stop_token_ids == (3, 5)
    assert (c.q_dim, c.kv_dim) == (96, 32)


def test_defaults_follow_the_reference():
    d = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 1, "hidden_size": 32, "num_attention_heads": 2,
         "intermediate_size": 64, "vocab_size": 50}
    c = config_from_dict(d)
    assert c.num_key_value_heads == 2          # kv heads default to heads
    assert c.head_dim == 16                    # hidden / heads
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0
    assert c.rope_scaling is None and c.tie_word_embeddings is False and c.stop_token_ids == ()
    assert c.rope_pairing == "half"


def test_explicit_head_dim_is_kept_apart_from_hidden_size():
    d = dict(TINY_A, head_dim=32)
    c = config_from_dict(d)
    assert c.head_dim == 32 and c.q_dim == 128 and c.hidden_size == 64


def test_missing_keys_are_all_named():
    with pytest.raises(ConfigError) as e:
        config_from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": 8})
    msg = str(e.value)
    for k in ("num_hidden_layers", "num_attention_heads", "intermediate_size", "vocab_size"):
        assert k in msg


@pytest.mark.parametrize("patch, word", [
    ({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"), ({"rope_scaling": {"type": "yarn"}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8}}, "low_freq_factor"), ({"attention_bias": True}, "bias"),
    ({"hidden_act": "gelu"}, "gelu"), ({"vocab_size": 0}, "vocab_size"), ({"hidden_size": "64"}, "integer"),
    ({"eos_token_id": "x"}, "eos_token_id"), ({"rope_pairing": "spiral"}, "rope_pairing"),
    ({"rms_norm_eps": 0}, "positive"), ({"torch_dtype": "int8"}, "torch_dtype"),
])
def test_bad_values_are_refused(patch, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict(dict(TINY_A, **patch))
    assert word in str(e.value)


def test_unknown_architecture_names_the_registered_ones():
    with pytest.raises(ConfigError) as e:
        config_from_dict(dict(TINY_A, architectures=["MambaForCausalLM"]))
    assert "MambaForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        config_from_dict({"hidden_size": 3})


def test_registry_accepts_and_drops_new_architectures():
    class Cfg(LlamaConfig):
        architecture = "ToyLlama"
    register_architecture("ToyLlama", Cfg)
    try:
        assert "ToyLlama" in registered_architectures()
        with pytest.raises(ConfigError):
            register_architecture("ToyLlama", Cfg)
        assert isinstance(config_from_dict(dict(TINY_A, architectures=["ToyLlama"])), Cfg)
    finally:
        unregister_architecture("ToyLlama")
    assert "ToyLlama" not in registered_architectures()


def test_round_trip_through_config_json(tmp_path):
    for d in (TINY_A, TINY_B):
        c = config_from_dict(d)
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        assert load_config(tmp_path) == c
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(tmp_path)
    with pytest.raises(ConfigError):
        load_config(tmp_path / "nowhere")


def test_the_model_is_data():
    c = config_from_dict(TINY_B)
    specs = c.layer_specs()
    assert len(specs) == 3
    s = specs[0]
    assert s.block == "pre_norm" and sorted(s.parts) == ["feed_forward", "feed_forward_norm", "mixer", "mixer_norm"]
    assert s.parts["mixer"].kind == "attention" and s.parts["feed_forward"].kind == "swiglu"
    assert s.parts["mixer_norm"].kind == "rmsnorm" and s.parts["mixer_norm"].family == "norm"
    assert s.parts["mixer"].args["n_heads"] == 3 and s.parts["mixer"].args["n_kv_heads"] == 1 and s.parts["mixer"].args["head_dim"] == 32
    assert s.parts["mixer"].args["position"].kind == "rope" and s.parts["mixer"].args["position"].args["theta"] == 500000.0
    assert s.parts["mixer_norm"].args["eps"] == 1e-6 and s.parts["feed_forward"].args["intermediate_size"] == 256
    assert [e.layer for e in c.schedule()] == [0, 1, 2] and [e.cache for e in c.schedule()] == [0, 1, 2]
    names = c.tensor_names()
    assert names["layers.2.mixer.k"] == "model.layers.2.self_attn.k_proj.weight"
    assert names["head.weight"] == "lm_head.weight"
    assert "head.weight" not in config_from_dict(TINY_A).tensor_names()   # tied: no separate head
