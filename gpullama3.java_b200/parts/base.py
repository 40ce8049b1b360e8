"""Interfaces of the parts a layer is put together from, their registries, and the step context
every part receives.

A part owns its sizes and constants as constructor parameters, declares its parameters
(``parameters()``), takes them as tensors (``load()``) and computes (``forward``).  No part knows
which model it is in: names of checkpoint tensors, the number of layers and the order of layers
live in the configuration.

Adding a part = subclass the interface below and call the matching ``register_*`` with a kind
name; a configuration then names that kind in its ``LayerSpec``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..weights.loader import ParamSpec


@dataclass
class StepContext:
    """One step's batch as the parts see it.  Tokens of all sequences are packed one after the
    other: sequence i owns rows cu_seqlens[i] .. cu_seqlens[i+1] of every [T, ...] activation.

    Host lists are for control flow (which kernel, how large a grid); device tensors (int32)
    are what kernels read."""
    dtype: torch.dtype               # float32 (true 32-bit run) or bfloat16
    device: torch.device
    n_seqs: int
    n_tokens: int
    slots: list[int]                 # cache slot of each sequence
    start_pos: list[int]             # tokens each sequence already has in the cache
    q_lens: list[int]                # tokens each sequence brings in this step
    all_decode: bool                 # every sequence brings exactly one token
    max_q_len: int
    max_kv_len: int                  # longest start_pos + q_len
    tokens: torch.Tensor             # [T] token ids
    positions: torch.Tensor          # [T] absolute position of each token in its sequence
    seq_ids: torch.Tensor            # [T] index (into this step's sequences) of each token
    cu_seqlens: torch.Tensor         # [n_seqs + 1]
    kv_lens: torch.Tensor            # [n_seqs] start_pos + q_len
    slots_dev: torch.Tensor          # [n_seqs]
    page_tables: list[torch.Tensor]  # per KV cache group: [n_seqs, width] physical page ids
    extras: dict = field(default_factory=dict)  # scratch a part may keep for the duration of a step


@dataclass
class ScaledRows:
    """Rows of an RMSNorm that is split between the product before it and the product after it: ``data`` holds
    x * weight (rounded to the run dtype) and row t still lacks its factor rsqrt(sum(partials[t]) / dim + eps).
    A part that says so (``takes_scaled_rows``) accepts this in place of normalised rows and lets its first
    product apply the factor; a part whose last product adds into the residual stream may be asked to leave
    the next norm in this form (``then_norm``).  Decode steps save two kernel launches per layer that way."""
    data: torch.Tensor       # [T, dim]
    partials: torch.Tensor   # float32 [T, P]
    eps: float
    dim: int

    @property
    def shape(self):
        return self.data.shape

    @property
    def device(self):
        return self.data.device


class Part:
    """Common face of all parts."""

    # True when the part's launches in a decode step depend only on device memory (the step
    # context's tensors, the cache), never on host-side numbers of the step such as slots or
    # lengths: only then may a decode step be recorded once and replayed as a CUDA graph.
    graph_safe: bool = False

    def parameters(self) -> dict[str, ParamSpec]:
        """Local parameter names -> shape and random-init kind."""
        return {}

    def load(self, tensors: dict[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        """Take the parameters (CPU or device tensors by local name), move and re-lay them out for
        the kernels.  ``dtype`` is the run's precision."""


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: torch.Tensor | None = None) -> torch.Tensor:
        """x: float32 residual stream [T, dim] -> normalised rows in ``out_dtype``; ``rows`` picks rows."""
        raise NotImplementedError

    def row_factor_form(self):
        """(weight [dim], eps, dim) if the norm is weight * x * f(row) with f = rsqrt(mean(x^2) + eps), so that
        it can be split between two products (see ScaledRows); None otherwise."""
        return None


class PositionEncoding(Part):
    """How positions enter a mixer.  The attention mixer asks for the rotary description."""
    rotary_dim: int = 0
    pairing: int = 0

    def inverse_frequencies(self, device) -> torch.Tensor:
        raise NotImplementedError


class Mixer(Part):
    """Mixes information between the tokens of a sequence."""

    def cache_need(self):
        """KVCacheNeed, StateNeed or None: what one run of this mixer keeps per sequence."""
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache, residual: torch.Tensor, writes_cache: bool = True) -> None:
        """x: normalised input [T, hidden] in the run dtype.  Adds the mixer's output to the float32
        ``residual`` [T, hidden] in place.  ``cache`` is the KVView/StateView of this run's entry.

        A mixer whose ``takes_scaled_rows(ctx)`` is true is also called with ``x`` a ScaledRows and with the
        keyword ``then_norm`` (a Norm or None); it returns the ScaledRows of that norm over the updated
        residual, or None if it left the norm to the caller."""
        raise NotImplementedError

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        return False


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        """Adds the feed-forward output of x [T, hidden] to ``residual`` in place.  With
        ``takes_scaled_rows(ctx)`` true: ``x`` may be a ScaledRows, ``then_norm`` as for a mixer."""
        raise NotImplementedError

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        return False


class Block(Part):
    """Arrangement of one layer's parts around the residual stream."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def children(self) -> dict[str, Part]:
        return {"mixer": self.mixer, "feed_forward": self.feed_forward, "mixer_norm": self.mixer_norm,
                "feed_forward_norm": self.feed_forward_norm}

    def forward(self, residual: torch.Tensor, ctx: StepContext, cache, writes_cache: bool = True) -> None:
        """Runs the layer on the float32 ``residual`` in place.  A block whose ``takes_scaled_rows(ctx)`` is
        true is also called with ``x_in`` (the ScaledRows of its first norm, or None) and ``then_norm`` (the
        first norm of the block that runs next, or None) and returns that norm's ScaledRows or None."""
        raise NotImplementedError

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        return False

    def first_norm(self) -> Norm | None:
        """The norm the block applies to the residual stream before anything else, if it starts that way."""
        return None


class PartRegistryError(KeyError):
    pass


_REGISTRIES: dict[str, dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}}


def _register(family: str, kind: str, cls: type, replace: bool) -> None:
    reg = _REGISTRIES[family]
    if kind in reg and not replace:
        raise PartRegistryError(f"{family} kind {kind!r} is already registered")
    reg[kind] = cls


def register_mixer(kind: str, cls: type, *, replace: bool = False) -> None:
    _register("mixer", kind, cls, replace)


def register_feed_forward(kind: str, cls: type, *, replace: bool = False) -> None:
    _register("feed_forward", kind, cls, replace)


def register_norm(kind: str, cls: type, *, replace: bool = False) -> None:
    _register("norm", kind, cls, replace)


def register_position_encoding(kind: str, cls: type, *, replace: bool = False) -> None:
    _register("position", kind, cls, replace)


def register_block(kind: str, cls: type, *, replace: bool = False) -> None:
    _register("block", kind, cls, replace)


def unregister(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


def registered(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])


def build_part(family: str, spec) -> Part:
    """Instantiate the registered class of ``spec.kind`` with ``spec.args``.  Arguments that are
    themselves part specs under the key ``position`` are built first."""
    from ..config.base import PartSpec

    reg = _REGISTRIES[family]
    if spec.kind not in reg:
        raise PartRegistryError(f"unknown {family} kind {spec.kind!r}; registered: {', '.join(sorted(reg)) or 'none'}")
    args = dict(spec.args)
    if isinstance(args.get("position"), PartSpec):
        args["position"] = build_part("position", args["position"])
    return reg[spec.kind](**args)
