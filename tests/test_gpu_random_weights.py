"""Random weights made on the device are the bits the CPU writes into a model folder from the same seed, so a model
filled in place (the benchmark's) can be reproduced by the plain implementation from a folder."""
import pytest
import torch

from conftest import TINY
from gpullama3.java_b200.config import config_from_dict
from gpullama3.java_b200.weights import random_checkpoint, write_random_model

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_device_and_cpu_make_the_same_bits(name, dtype):
    cfg_json, norm_std = TINY[name]
    cfg = config_from_dict(cfg_json)
    on_cpu = dict(random_checkpoint(cfg, 11, dtype=dtype, norm_std=norm_std))
    on_gpu = dict(random_checkpoint(cfg, 11, dtype=dtype, norm_std=norm_std, device="cuda"))
    assert list(on_cpu) == list(on_gpu)
    for n in on_cpu:
        assert on_gpu[n].dtype == on_cpu[n].dtype and torch.equal(on_gpu[n].cpu(), on_cpu[n]), n
    other = dict(random_checkpoint(cfg, 12, dtype=dtype, norm_std=norm_std, device="cuda"))
    assert not torch.equal(other["model.embed_tokens.weight"], on_gpu["model.embed_tokens.weight"])


def test_a_long_tensor_in_one_launch_equals_the_cpu_in_many_passes():
    from gpullama3.java_b200.kernels import ops
    from gpullama3.java_b200.weights.random_init import normal_scale, random_values, tensor_key

    key, n = tensor_key(3, "some.weight"), 1_000_003
    out = torch.empty(n, dtype=torch.float32, device="cuda")
    ops.random_fill(out, key, float(normal_scale(0.02)), 0.0)
    assert torch.equal(out.cpu(), random_values(key, n, 0.02))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_filled_in_place_gives_the_logits_of_its_folder(tmp_path, dtype):
    from gpullama3.java_b200.engine.api import Engine, SequenceInput

    cfg_json, norm_std = TINY["B"]
    folder = write_random_model(config_from_dict(cfg_json), 5, tmp_path / "m", norm_std=norm_std)
    a = Engine.from_folder(folder, dtype=dtype, max_tokens=64 * 2, max_batch=2)
    b = Engine.from_random(cfg_json, 5, dtype=dtype, norm_std=norm_std, max_tokens=64 * 2, max_batch=2)
    prompt = list(range(3, 40))
    la = a.step([SequenceInput(a.cache.acquire(), prompt, list(range(len(prompt))))])
    lb = b.step([SequenceInput(b.cache.acquire(), prompt, list(range(len(prompt))))])
    assert torch.equal(la, lb)
