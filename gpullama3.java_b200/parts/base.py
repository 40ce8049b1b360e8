"""Interfaces of the parts a layer is put together from, their registries, and the step context
every part receives.

A part owns its sizes and constants as constructor parameters, declares its parameters
(``parameters()``), takes them as tensors (``load()``) and computes (``forward``).  No part knows
which model it is in: names of checkpoint tensors, the number of layers and the order of layers
live in the configuration.

Adding a part = subclass the interface below and call the matching ``register_*`` (or
``register_part`` with a family name of one's own) with a kind name; a configuration then names
family and kind in a ``PartSpec``.
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
    page_tables: list[torch.Tensor]  # per paged cache group: [n_seqs, width] physical page ids
    # per paged cache group: the longest sequence this step's launches must be right for.  A step that runs
    # once needs no more than max_kv_len; a recorded decode step is replayed while its page tables can address
    # the sequences, so a part that shapes its launch by length (spans of keys) shapes it for this number.
    kv_capacity: list[int] = field(default_factory=list)
    extras: dict = field(default_factory=dict)  # scratch a part may keep for the duration of a step
    workspace: object = None         # where intermediate tensors of this pass come from (None: the allocator)

    def empty(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """An uninitialised device tensor that lives until the block that asked for it has run (the model gives
        a block's pieces back after it); what must live longer (logits, anything handed to the next block) is
        taken from ``torch.empty``."""
        if self.workspace is not None:
            return self.workspace.take(shape, dtype)
        return torch.empty(tuple(shape), dtype=dtype, device=self.device)

    def capacity(self, group: int) -> int:
        return self.kv_capacity[group] if group < len(self.kv_capacity) else self.max_kv_len


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

    # True when tokens appended behind a pass's own tokens change nothing that the own tokens' results or any later
    # step depend on: per-token parts, and mixers whose only memory is a cache that is read causally and written at
    # each token's own position.  Only then may a short prompt run as a recorded pass padded to a whole page
    # (a mixer that folds every token it sees into a state of fixed size is not: the padding would enter the state).
    pad_safe: bool = False

    def parameters(self) -> dict[str, ParamSpec]:
        """Local parameter names -> shape and random-init kind."""
        return {}

    def load(self, tensors: dict[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        """Take the parameters (CPU or device tensors by local name), move and re-lay them out for
        the kernels.  ``dtype`` is the run's precision."""

    def children(self) -> dict[str, "Part"]:
        """Parts this part was built with, by the names it gives them.  Their parameters are declared and
        loaded under ``<this part's path>.<name>``; the part itself only declares its own."""
        return {}


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: torch.Tensor | None = None, alloc=None) -> torch.Tensor:
        """x: float32 residual stream [T, dim] -> normalised rows in ``out_dtype``; ``rows`` picks rows.
        ``alloc(shape, dtype)``: where the result comes from (a step's ``ctx.empty``; default: the allocator)."""
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
    """Arrangement of one layer's parts around the residual stream.  A block's constructor takes its parts
    by keyword, under names of its own choosing (the configuration's ``LayerSpec.parts`` uses the same names)
    and hands them to ``Block.__init__``; which parts a layer has is therefore the block's business alone."""

    def __init__(self, **parts: Part):
        self.parts: dict[str, Part] = dict(parts)
        for name, part in parts.items():
            setattr(self, name, part)

    def children(self) -> dict[str, Part]:
        return dict(self.parts)

    def cache_need(self):
        """What one run of this block keeps per sequence: the need of its one part that has any."""
        needs = [(n, p.cache_need()) for n, p in self.parts.items() if hasattr(p, "cache_need")]
        needs = [(n, need) for n, need in needs if need is not None]
        if len(needs) > 1:
            raise ValueError("a block with several caching parts (" + ", ".join(n for n, _ in needs) +
                             ") must say itself what one run of it keeps (override cache_need)")
        return needs[0][1] if needs else None

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


def all_parts(root: Part, prefix: str = "") -> dict[str, Part]:
    """Every part below ``root`` by dotted path (``mixer``, ``mixer.position``), parents before children."""
    out: dict[str, Part] = {}
    for name, part in root.children().items():
        path = f"{prefix}{name}"
        out[path] = part
        out.update(all_parts(part, path + "."))
    return out


class PartRegistryError(KeyError):
    pass


_REGISTRIES: dict[str, dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}}


def register_part(family: str, kind: str, cls: type, *, replace: bool = False) -> None:
    """Register ``cls`` as ``kind`` of ``family``; a family that does not exist yet is created."""
    reg = _REGISTRIES.setdefault(family, {})
    if kind in reg and not replace:
        raise PartRegistryError(f"{family} kind {kind!r} is already registered")
    reg[kind] = cls


def register_mixer(kind: str, cls: type, *, replace: bool = False) -> None:
    register_part("mixer", kind, cls, replace=replace)


def register_feed_forward(kind: str, cls: type, *, replace: bool = False) -> None:
    register_part("feed_forward", kind, cls, replace=replace)


def register_norm(kind: str, cls: type, *, replace: bool = False) -> None:
    register_part("norm", kind, cls, replace=replace)


def register_position_encoding(kind: str, cls: type, *, replace: bool = False) -> None:
    register_part("position", kind, cls, replace=replace)


def register_block(kind: str, cls: type, *, replace: bool = False) -> None:
    register_part("block", kind, cls, replace=replace)


def unregister(family: str, kind: str) -> None:
    _REGISTRIES.get(family, {}).pop(kind, None)


def registered(family: str) -> list[str]:
    return sorted(_REGISTRIES.get(family, {}))


def _registered_class(family: str, kind: str) -> type:
    reg = _REGISTRIES.get(family)
    if reg is None:
        raise PartRegistryError(f"unknown part family {family!r}; families: {', '.join(sorted(_REGISTRIES))}")
    if kind not in reg:
        raise PartRegistryError(f"unknown {family} kind {kind!r}; registered: {', '.join(sorted(reg)) or 'none'}")
    return reg[kind]


def _built(value):
    """``value`` with every PartSpec in it (also inside lists, tuples and dicts) replaced by the built part."""
    from ..config.base import PartSpec

    if isinstance(value, PartSpec):
        return build_part(value)
    if isinstance(value, (list, tuple)):
        return type(value)(_built(v) for v in value)
    if isinstance(value, dict):
        return {k: _built(v) for k, v in value.items()}
    return value


def build_part(spec) -> Part:
    """Instantiate the class registered as ``spec.kind`` in ``spec.family`` with ``spec.args``; arguments that
    are part specs themselves are built first, whatever their key."""
    cls = _registered_class(spec.family, spec.kind)
    return cls(**{k: _built(v) for k, v in spec.args.items()})


def build_block(spec) -> Block:
    """The block of a ``LayerSpec``: its registered class, given the layer's built parts by name."""
    cls = _registered_class("block", spec.block)
    try:
        return cls(**{name: build_part(p) for name, p in spec.parts.items()})
    except TypeError as e:
        raise PartRegistryError(f"block kind {spec.block!r} does not take the parts "
                                f"{sorted(spec.parts)}: {e}") from e
