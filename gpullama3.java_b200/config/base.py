"""What every architecture's configuration tells the engine.

A configuration is a typed record read from the architecture's own ``config.json`` keys.  Beyond
its numbers it answers four questions, all as data, so that the engine holds no size or constant
of any model:

* ``layer_specs()``  which block arrangement each layer has and which parts that block is given, by
  the names the block itself uses (a pre-norm block takes ``mixer``, ``feed_forward`` and two norms;
  another block may take fewer or other parts), each with its parameters (sizes, eps, window, rope
  constants);
* ``schedule()``     in which order layers run; a layer may appear twice, and an entry may read
  the cache that another entry writes;
* ``tensor_names()`` under which checkpoint name each parameter of each part is stored;
* the embedding, final norm and output head (sizes, tying).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """config.json is missing, malformed, or describes a model the engine cannot build."""


@dataclass(frozen=True)
class PartSpec:
    """One part: the family it belongs to (``mixer``, ``feed_forward``, ``norm``, ``position``, ...), the kind
    registered in that family, and the keyword arguments it is built with.  An argument may itself be a
    PartSpec (an attention mixer's position encoding, a norm inside a mixer): it is built first and handed
    over as a part."""
    family: str
    kind: str
    args: dict[str, Any] = field(default_factory=dict)

    def with_args(self, **changes) -> "PartSpec":
        return PartSpec(self.family, self.kind, {**self.args, **changes})


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the registered block kind and the parts it is built from, under the names that block's
    constructor takes.  Nothing else fixes which parts a layer has."""
    block: str
    parts: dict[str, PartSpec]

    def with_parts(self, **changes: PartSpec) -> "LayerSpec":
        return LayerSpec(self.block, {**self.parts, **changes})


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache`` names the cache entry the mixer uses; two schedule entries
    with the same ``cache`` share keys and values, and only the one with ``writes_cache`` stores
    them.  ``cache`` is None for a mixer that keeps nothing."""
    layer: int
    cache: int | None
    writes_cache: bool = True


def default_schedule(n_layers: int) -> list[ScheduleEntry]:
    return [ScheduleEntry(layer=i, cache=i) for i in range(n_layers)]


class ModelConfig:
    """Base of all typed configurations.  Subclasses are dataclasses that implement
    ``from_dict`` (reading config.json keys), ``to_dict`` (writing them back), ``layer_specs``,
    ``tensor_names`` and the few attributes below."""

    architecture: str = ""
    hidden_size: int
    vocab_size: int
    tie_word_embeddings: bool
    stop_token_ids: tuple[int, ...] = ()

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    def layer_specs(self) -> list[LayerSpec]:
        raise NotImplementedError

    def schedule(self) -> list[ScheduleEntry]:
        return default_schedule(len(self.layer_specs()))

    def final_norm(self) -> PartSpec:
        raise NotImplementedError

    def tensor_names(self) -> dict[str, str]:
        """Map from a part's parameter path (``layers.3.mixer.q``, ``embedding.table``,
        ``final_norm.weight``, ``head.weight``) to its checkpoint tensor name."""
        raise NotImplementedError

    def max_sequence_length(self) -> int | None:
        """The longest sequence (prompt and generated tokens together) the model is meant for, if the
        configuration gives one; generation stops there even when the cache has room for more."""
        return None

    def optional_tensor_names(self) -> set[str]:
        """Checkpoint tensors that may be present without being read (some exporters store the output head
        of a tied model a second time); anything else that the model does not declare is reported."""
        return set()

    def init_std(self) -> float:
        """Standard deviation of random matrices in the random-weights mode."""
        return 0.02


def read_config_json(model_dir: str | Path) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {model_dir}")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d


def require_keys(d: dict, keys: list[str], what: str) -> None:
    missing = [k for k in keys if k not in d or d[k] is None]
    if missing:
        raise ConfigError(f"{what}: missing key(s) {', '.join(missing)}")


def as_int(d: dict, key: str, *, minimum: int = 1) -> int:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config key {key!r} must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config key {key!r} must be >= {minimum}, got {v}")
    return v


def as_float(d: dict, key: str) -> float:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config key {key!r} must be a number, got {v!r}")
    return float(v)
