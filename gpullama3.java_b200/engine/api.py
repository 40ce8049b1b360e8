"""The Python entry point: an ``Engine`` holds a loaded model, its cache, the step function and the
generation loop.

    engine = Engine.from_folder("model_dir", dtype="bfloat16", max_tokens=32768)
    outputs = engine.generate([[1, 2, 3], [4, 5]], max_new_tokens=16)          # greedy
    outputs = engine.generate(prompts, max_new_tokens=16, temperature=0.8, seed=1)

Token ids go in and come out as Python lists; everything between runs on the GPU."""
from __future__ import annotations

from pathlib import Path

import torch

from ..cache.pages import PAGE_TOKENS
from ..config.base import ModelConfig, read_config_json
from ..config.registry import architecture_of
from ..sampling.sampler import Sampler, SamplingParams
from .generate import GenerationResult, Generator
from .step import SequenceInput, StepFunction

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _resolve_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {dtype!r}") from None


def resolve_max_length(config: ModelConfig, cache_tokens: int, asked: int | None = None) -> int:
    """The longest sequence generation allows: what was asked for, else the smaller of what the cache holds
    and the configuration's own context length."""
    if asked is not None:
        if asked < 1:
            raise ValueError(f"max_length must be positive, got {asked}")
        return int(asked)
    limit = config.max_sequence_length()
    return cache_tokens if limit is None else min(cache_tokens, int(limit))


def read_stop_ids(model_dir: str | Path, config: ModelConfig) -> tuple[int, ...]:
    """Stop token ids of a model folder: ``eos_token_id`` (an integer or a list) of generation_config.json when
    that file has one, else the configuration's own.  The reference takes them from its chat format
    (model/format/LlamaChatFormat.java:30 of the reference project); a model folder states them in these files."""
    import json

    path = Path(model_dir) / "generation_config.json"
    if path.is_file():
        try:
            eos = json.loads(path.read_text()).get("eos_token_id")
        except (json.JSONDecodeError, AttributeError) as e:
            raise ValueError(f"{path} is not a JSON object: {e}") from e
        if isinstance(eos, int) and not isinstance(eos, bool):
            return (eos,)
        if isinstance(eos, list) and eos and all(isinstance(t, int) and not isinstance(t, bool) for t in eos):
            return tuple(eos)
        if eos is not None:
            raise ValueError(f"{path}: eos_token_id must be an integer or a list of integers, got {eos!r}")
    return tuple(config.stop_token_ids)


class _LoopStep:
    """The step function as the generation loop uses it: the loop samples from a step's logits before it runs
    the next step, so the logits need not be copied; decode steps may come back as drawn tokens directly, and may be launched
    one ahead of the tokens the host has read."""

    def __init__(self, step_fn: StepFunction):
        self.step_fn = step_fn
        self.decode_and_sample = step_fn.decode_and_sample
        self.decode_ahead, self.collect, self.abandon = step_fn.decode_ahead, step_fn.collect, step_fn.abandon

    def __call__(self, inputs):
        return self.step_fn(inputs, reuse_output=True)


class Engine:
    def __init__(self, model, *, max_tokens: int = 32768, max_batch: int = 64, max_length: int | None = None):
        if not torch.cuda.is_available() or model.device.type != "cuda":
            raise RuntimeError("the engine needs a CUDA device; it has no CPU path")
        self.model = model
        self.config: ModelConfig = model.config
        self.cache = model.new_cache(max_tokens, max_slots=max(max_batch, 1))
        self.step_fn = StepFunction(model, self.cache)
        self.max_length = resolve_max_length(self.config, self.cache.n_pages * PAGE_TOKENS, max_length)
        self.stop_ids: tuple[int, ...] = tuple(self.config.stop_token_ids)
        self.generator = Generator(_LoopStep(self.step_fn), self.cache, Sampler, max_batch=max_batch,
                                   max_length=self.max_length)

    # ---- construction
    @classmethod
    def from_folder(cls, model_dir: str | Path, *, dtype="bfloat16", device="cuda", **kw) -> "Engine":
        d = read_config_json(model_dir)
        arch = architecture_of(d)
        model = arch.model_factory(arch.config_class.from_dict(d), _resolve_dtype(dtype), device)
        model.load_folder(model_dir)
        engine = cls(model, **kw)
        engine.stop_ids = read_stop_ids(model_dir, engine.config)
        return engine

    @classmethod
    def from_random(cls, config: ModelConfig | dict, seed: int = 0, *, dtype="bfloat16", device="cuda",
                    norm_std: float = 0.0, **kw) -> "Engine":
        if isinstance(config, dict):
            arch = architecture_of(config)
            config = arch.config_class.from_dict(config)
        else:
            arch = architecture_of({"architectures": [config.architecture]})
        model = arch.model_factory(config, _resolve_dtype(dtype), device)
        model.load_random(seed, norm_std=norm_std)
        return cls(model, **kw)

    # ---- use
    def generate(self, prompts: list[list[int]], max_new_tokens: int = 16, *, temperature: float = 0.0,
                 top_p: float = 1.0, seed: int = 0, stop_ids=None, on_token=None,
                 return_results: bool = False):
        """Generated token ids per prompt (the stop token included when one ended the sequence)."""
        if stop_ids is None:
            stop_ids = self.stop_ids
        results = self.generator.generate([list(p) for p in prompts], max_new_tokens,
                                          SamplingParams(temperature, top_p, seed), stop_ids, on_token)
        return results if return_results else [r.tokens for r in results]

    @property
    def last_metrics(self):
        return self.generator.last_metrics

    def step(self, inputs: list[SequenceInput]) -> torch.Tensor | None:
        return self.step_fn(inputs)


__all__ = ["Engine", "GenerationResult", "SequenceInput", "SamplingParams"]
