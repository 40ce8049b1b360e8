"""Random-weights mode: tensors from a configuration and a seed, and a model folder written from
them.  Each tensor's values depend only on (seed, checkpoint name), not on the order of creation,
so a folder and an in-memory model made from the same seed hold the same numbers."""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from ..config.base import ModelConfig
from .loader import ParamSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(name: str, spec: ParamSpec, seed: int, std: float, norm_std: float, dtype: torch.dtype,
                  device: str | torch.device = "cpu") -> torch.Tensor:
    """One tensor of the random-weights mode, generated in float32 and rounded once to ``dtype``."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if spec.init == "matrix":
        t = torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32) * std
    elif spec.init == "norm":
        t = torch.ones(spec.shape, device=device, dtype=torch.float32)
        if norm_std:
            t = t + torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32) * norm_std
    elif spec.init == "zeros":
        t = torch.zeros(spec.shape, device=device, dtype=torch.float32)
    elif spec.init == "int_table":
        return torch.zeros(spec.shape, device=device, dtype=torch.int32)
    else:
        raise ValueError(f"unknown init kind {spec.init!r} for {name}")
    return t.to(dtype)


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
