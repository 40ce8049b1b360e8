"""Random-weights mode: tensors from a configuration and a seed, and a model folder written from
them.

Every element is a fixed function of (seed, checkpoint name of its tensor, its index in the
tensor): it does not depend on the order in which tensors are made, on the device, or on how a
tensor is cut into chunks.  The function is written twice, here with numpy for the CPU (model
folders, the tests' plain implementation) and in ``csrc/random_init.cu`` for the device
(``CausalLM.load_random``, the benchmark's models), and both give the same bits: the random part
is integer arithmetic, followed by one exact conversion, one multiplication and one addition in
float32, then one rounding to the storage type.

value(i) = offset + scale * (s(i) - 524280).  s(i) is the sum of the sixteen 16-bit fields of
outputs 4i .. 4i + 3 of the splitmix64 sequence whose start is the first eight bytes of
SHA-256("<seed>:<name>"); the sum of sixteen uniform numbers is normal to a good approximation
(mean 524280, bounded at 6.9 standard deviations).  ``scale`` = std / sqrt(16 (65536^2 - 1) / 12)."""
from __future__ import annotations

import hashlib
import json
import math
from pathlib import Path

import numpy as np
import torch

from ..config.base import ModelConfig
from .loader import ParamSpec
from .safetensors_io import write_safetensors

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1, _M2 = np.uint64(0xBF58476D1CE4E5B9), np.uint64(0x94D049BB133111EB)
_SUM_MEAN = 524280                                          # 16 * 32767.5
_SUM_SIGMA = math.sqrt(16 * (65536.0 ** 2 - 1.0) / 12.0)    # of the sum of sixteen 16-bit uniform numbers
_CHUNK = 1 << 17   # elements per pass of the numpy version: its temporaries stay in the cache


def tensor_key(seed: int, name: str) -> int:
    """Start of the tensor's number sequence: 64 bits of SHA-256("<seed>:<name>")."""
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _centred_sums(key: int, start: int, n: int) -> np.ndarray:
    """s(i) - 524280 for i in [start, start + n), as int32."""
    with np.errstate(over="ignore"):
        i = np.arange(start, start + n, dtype=np.uint64)
        total = np.zeros(n, dtype=np.uint32)
        for r in range(4):
            z = np.uint64(key) + (np.uint64(4) * i + np.uint64(r + 1)) * _GOLDEN
            z = (z ^ (z >> np.uint64(30))) * _M1
            z = (z ^ (z >> np.uint64(27))) * _M2
            z = z ^ (z >> np.uint64(31))
            for shift in (0, 16, 32, 48):
                total += ((z >> np.uint64(shift)) & np.uint64(0xFFFF)).astype(np.uint32)
    return total.astype(np.int32) - np.int32(_SUM_MEAN)


def normal_scale(std: float) -> np.float32:
    return np.float32(std / _SUM_SIGMA)


def random_values(key: int, n: int, std: float, offset: float = 0.0) -> torch.Tensor:
    """float32 [n] on the CPU: offset + N(0, std) by the function above."""
    out = np.empty(n, dtype=np.float32)
    scale, off = normal_scale(std), np.float32(offset)
    for start in range(0, n, _CHUNK):
        m = min(_CHUNK, n - start)
        out[start:start + m] = off + _centred_sums(key, start, m).astype(np.float32) * scale
    return torch.from_numpy(out)


def random_tensor(name: str, spec: ParamSpec, seed: int, std: float, norm_std: float, dtype: torch.dtype,
                  device: str | torch.device = "cpu") -> torch.Tensor:
    """One tensor of the random-weights mode, in float32 and rounded once to ``dtype``; on a CUDA device it is
    made there by the kernel, with the bits the CPU would give."""
    device = torch.device(device)
    if spec.init == "int_table":
        return torch.zeros(spec.shape, device=device, dtype=torch.int32)
    if spec.init == "zeros" or (spec.init == "norm" and not norm_std):
        return torch.full(spec.shape, 0.0 if spec.init == "zeros" else 1.0, device=device, dtype=dtype)
    if spec.init == "matrix":
        s, offset = std, 0.0
    elif spec.init == "norm":
        s, offset = norm_std, 1.0
    else:
        raise ValueError(f"unknown init kind {spec.init!r} for {name}")
    key, n = tensor_key(seed, name), math.prod(spec.shape)
    if device.type == "cuda":
        from ..kernels import ops
        out = torch.empty(spec.shape, dtype=dtype if dtype in (torch.float32, torch.bfloat16) else torch.float32,
                          device=device)
        ops.random_fill(out, key, float(normal_scale(s)), offset)
        return out.to(dtype)
    return random_values(key, n, s, offset).reshape(spec.shape).to(dtype)


def random_checkpoint(config: ModelConfig, seed: int, *, dtype: torch.dtype = torch.bfloat16, norm_std: float = 0.0,
                      norm_dtype: torch.dtype | None = None, device: str | torch.device = "cpu"):
    """Yield (checkpoint name, tensor) for every parameter the model of ``config`` declares."""
    from ..engine.model import parameter_specs_by_checkpoint_name

    for name, spec in parameter_specs_by_checkpoint_name(config).items():
        d = norm_dtype if (spec.init == "norm" and norm_dtype is not None) else dtype
        yield name, random_tensor(name, spec, seed, config.init_std(), norm_std, d, device)


def write_random_model(config: ModelConfig, seed: int, out_dir: str | Path, *, dtype: torch.dtype = torch.bfloat16,
                       norm_std: float = 0.0, norm_dtype: torch.dtype | None = None) -> Path:
    """Write ``config.json`` and ``model.safetensors`` of a randomly initialised model."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    tensors = dict(random_checkpoint(config, seed, dtype=dtype, norm_std=norm_std, norm_dtype=norm_dtype))
    write_safetensors(out / "model.safetensors", tensors,
                      metadata={"format": "pt", "random_seed": seed, "norm_std": norm_std})
    return out
