"""Weights: the safetensors container, binding by name, errors, the random-weights mode (no GPU)."""
import json
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B, make_model_dir
from gpullama3.java_b200.config import config_from_dict
from gpullama3.java_b200.engine.model import CausalLM, parameter_specs_by_checkpoint_name
from gpullama3.java_b200.weights import (SafetensorsFile, WeightError, load_checkpoint_tensors, open_model_files,
                                         random_checkpoint, storage_dtype, write_random_model, write_safetensors)


def test_container_round_trip_both_ways(tmp_path):
    from safetensors.torch import load_file, save_file

    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
         "c": torch.randn(4, dtype=torch.float32), "d": torch.randn(2, 2).to(torch.float16)}
    write_safetensors(tmp_path / "ours.safetensors", t)
    theirs = load_file(str(tmp_path / "ours.safetensors"))
    assert set(theirs) == set(t) and all(torch.equal(theirs[k], t[k]) for k in t)
    save_file(t, str(tmp_path / "theirs.safetensors"))
    f = SafetensorsFile(tmp_path / "theirs.safetensors")
    assert sorted(f.names()) == sorted(t)
    for k in t:
        assert f.dtype(k) == t[k].dtype and f.shape(k) == tuple(t[k].shape) and torch.equal(f.tensor(k), t[k])


def test_malformed_files_are_refused(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(WeightError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 10**9) + b"{}")
    with pytest.raises(WeightError, match="header length"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 5) + b"{oops")
    with pytest.raises(WeightError, match="JSON"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)      # data region shorter than claimed
    with pytest.raises(WeightError, match="claims bytes"):
        SafetensorsFile(p)
    with pytest.raises(WeightError, match="does not exist"):
        SafetensorsFile(tmp_path / "absent.safetensors")
    with pytest.raises(WeightError, match="no model.safetensors"):
        open_model_files(tmp_path / "empty_dir_that_is_not_there")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = config_from_dict(TINY_A)
    tensors = dict(random_checkpoint(cfg, 0))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    write_safetensors(tmp_path / "model.safetensors", tensors)
    model = CausalLM(cfg, torch.float32, "cpu")
    with pytest.raises(WeightError) as e:
        model.load_folder(tmp_path)
    msg = str(e.value)
    assert "missing (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "unexpected (1)" in msg and "q_proj.bias" in msg
    assert "wrong shape (1)" in msg and "k_proj.weight is [16, 64], expected [32, 64]" in msg


def test_tied_model_ignores_a_stored_head_and_untied_needs_it(tmp_path):
    cfg = config_from_dict(TINY_A)
    tensors = dict(random_checkpoint(cfg, 0))
    assert "lm_head.weight" not in tensors
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(tmp_path / "model.safetensors", tensors)
    expected = {n: s.shape for n, s in parameter_specs_by_checkpoint_name(cfg).items()}
    load_checkpoint_tensors(tmp_path, expected, torch.bfloat16, optional={"lm_head.weight"})
    assert "lm_head.weight" in parameter_specs_by_checkpoint_name(config_from_dict(TINY_B))


def test_storage_policy():
    bf, f32 = torch.bfloat16, torch.float32
    assert storage_dtype(torch.bfloat16, bf) == bf and storage_dtype(torch.float16, bf) == bf
    assert storage_dtype(torch.float32, bf) == f32          # a tensor stored in 32 bits stays so
    assert storage_dtype(torch.int64, bf) == torch.int32 and storage_dtype(torch.uint8, f32) == torch.int32
    assert storage_dtype(torch.bfloat16, f32) == f32 and storage_dtype(torch.float16, f32) == f32


def test_load_keeps_32_bit_norm_weights(tmp_path):
    d = make_model_dir(tmp_path, TINY_B, seed=2, norm_std=0.1, norm_dtype=torch.float32)
    cfg = config_from_dict(json.loads((d / "config.json").read_text()))
    expected = {n: s.shape for n, s in parameter_specs_by_checkpoint_name(cfg).items()}
    t = load_checkpoint_tensors(d, expected, torch.bfloat16)
    assert t["model.norm.weight"].dtype == torch.float32
    assert t["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    t32 = load_checkpoint_tensors(d, expected, torch.float32)
    assert all(v.dtype == torch.float32 for v in t32.values())
    assert torch.equal(t32["model.layers.0.self_attn.q_proj.weight"], t["model.layers.0.self_attn.q_proj.weight"].float())


def test_random_weights_mode_is_reproducible(tmp_path):
    cfg = config_from_dict(TINY_B)
    a = write_random_model(cfg, 7, tmp_path / "a", norm_std=0.1)
    b = write_random_model(cfg, 7, tmp_path / "b", norm_std=0.1)
    c = write_random_model(cfg, 8, tmp_path / "c", norm_std=0.1)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    assert json.loads((a / "config.json").read_text())["architectures"] == ["LlamaForCausalLM"]
    f = SafetensorsFile(a / "model.safetensors")
    w = f.tensor("model.layers.0.mlp.gate_proj.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    n = f.tensor("model.layers.1.input_layernorm.weight").float()
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.05 < float(n.std()) < 0.15
    ones = SafetensorsFile(write_random_model(config_from_dict(TINY_A), 1, tmp_path / "d") / "model.safetensors")
    assert torch.equal(ones.tensor("model.norm.weight").float(), torch.ones(64))


def test_random_values_depend_on_seed_name_and_index_only():
    from gpullama3.java_b200.weights.random_init import random_values, tensor_key

    key = tensor_key(7, "model.layers.0.mlp.gate_proj.weight")
    assert key != tensor_key(8, "model.layers.0.mlp.gate_proj.weight") != tensor_key(7, "model.layers.1.mlp.gate_proj.weight")
    a = random_values(key, 300_000, 0.02)                    # more than one pass of the generator
    assert torch.equal(a[:1000], random_values(key, 1000, 0.02))              # a prefix is the same numbers
    assert not torch.equal(a[:1000], random_values(key + 1, 1000, 0.02))
    assert abs(float(a.mean())) < 2e-4 and abs(float(a.std()) - 0.02) < 2e-4
    z = a.double() / 0.02
    assert abs(float((z ** 4).mean()) - 3.0) < 0.1 and float(z.abs().max()) < 6.93       # near normal, bounded
    shifted = random_values(key, 1000, 0.1, offset=1.0)
    assert abs(float(shifted.mean()) - 1.0) < 0.02
    # first values, fixed here so that a change of the function does not pass unnoticed
    first = random_values(tensor_key(0, "w"), 4, 1.0)
    assert first.dtype == torch.float32 and torch.isfinite(first).all()
    assert torch.equal(first, random_values(tensor_key(0, "w"), 4, 1.0))


def test_sharded_folder(tmp_path):
    cfg = config_from_dict(TINY_A)
    tensors = dict(random_checkpoint(cfg, 0))
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(tmp_path / "s1.safetensors", {n: tensors[n] for n in names[:half]})
    write_safetensors(tmp_path / "s2.safetensors", {n: tensors[n] for n in names[half:]})
    wm = {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    expected = {n: s.shape for n, s in parameter_specs_by_checkpoint_name(cfg).items()}
    got = load_checkpoint_tensors(tmp_path, expected, torch.bfloat16)
    assert all(torch.equal(got[n], tensors[n]) for n in names)
    wm[names[0]] = "s2.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    with pytest.raises(WeightError, match="does not hold"):
        load_checkpoint_tensors(tmp_path, expected, torch.bfloat16)
