"""The decoder assembled from parts: embedding, a schedule of blocks, final norm, output head.

Everything that differs between models is data from the configuration: which parts each layer
has (``layer_specs``), in which order layers run and whose cache each run uses (``schedule``),
and the checkpoint name of every parameter (``tensor_names``).  The computation follows
inference/InferenceCore.java:58-180 of the reference project, for a packed batch of tokens
instead of one token."""
from __future__ import annotations

from pathlib import Path

import torch

from ..cache.sequence_cache import SequenceCache
from ..config.base import ConfigError, ModelConfig, ScheduleEntry
from ..parts.base import Block, Part, StepContext, all_parts, build_block, build_part
from ..parts.embedding import OutputHead, TokenEmbedding
from ..weights.loader import ParamSpec, load_checkpoint_tensors
from ..weights.safetensors_io import WeightError


class CausalLM:
    def __init__(self, config: ModelConfig, dtype: torch.dtype = torch.bfloat16, device="cuda"):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ConfigError(f"the engine runs in float32 or bfloat16, not {dtype}")
        self.config, self.dtype, self.device = config, dtype, torch.device(device)
        self.embedding = TokenEmbedding(config.vocab_size, config.hidden_size)
        self.blocks: list[Block] = [build_block(s) for s in config.layer_specs()]
        self.final_norm = build_part(config.final_norm())
        self.head = OutputHead(config.vocab_size, config.hidden_size,
                               tied_to=self.embedding if config.tie_word_embeddings else None)
        self.schedule: list[ScheduleEntry] = list(config.schedule())
        self._check_schedule()
        self.loaded = False

    # ---- structure
    def _check_schedule(self) -> None:
        writers: dict[int, int] = {}
        needs: dict[int, object] = {}
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.blocks)):
                raise ConfigError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.blocks)}")
            need = self.blocks[e.layer].cache_need()
            if need is None:
                if e.cache is not None:
                    raise ConfigError(f"schedule entry {i}: layer {e.layer} keeps no cache but the entry names cache {e.cache}")
                continue
            if e.cache is None:
                raise ConfigError(f"schedule entry {i}: layer {e.layer} needs a cache entry")
            if e.cache in needs and needs[e.cache] != need:
                raise ConfigError(f"schedule entry {i}: cache {e.cache} is shared by mixers with different needs")
            needs[e.cache] = need
            if e.writes_cache:
                if e.cache in writers:
                    raise ConfigError(f"cache {e.cache} is written by schedule entries {writers[e.cache]} and {i}")
                writers[e.cache] = i
            elif e.cache not in writers:
                raise ConfigError(f"schedule entry {i} reads cache {e.cache} before any entry writes it")
        self._cache_needs = needs

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model may be recorded once and replayed as a CUDA graph."""
        return all(p.graph_safe for p in self.named_parts().values()) and all(b.graph_safe for b in self.blocks)

    @property
    def pad_safe(self) -> bool:
        """Whether a short prompt may run as a recorded pass padded with tokens that are never committed."""
        return all(p.pad_safe for p in self.named_parts().values()) and all(getattr(b, "pad_safe", False) for b in self.blocks)

    def cache_needs(self) -> dict[int, object]:
        """Cache entry id -> the need (KVCacheNeed, StateNeed, or a type of the mixer's own) of the runs that use it."""
        return dict(self._cache_needs)

    def named_parts(self) -> dict[str, Part]:
        """Every part by its path: ``embedding``, ``layers.3.mixer``, ``layers.3.mixer.position``, ..."""
        parts: dict[str, Part] = {"embedding": self.embedding}
        parts.update(all_parts(self.embedding, "embedding."))
        for i, b in enumerate(self.blocks):
            parts.update(all_parts(b, f"layers.{i}."))
        for name, part in (("final_norm", self.final_norm), ("head", self.head)):
            parts[name] = part
            parts.update(all_parts(part, name + "."))
        return parts

    def parameter_specs(self) -> dict[str, ParamSpec]:
        """Parameter path (``layers.0.mixer.q``) -> spec, for every part."""
        return {f"{path}.{local}": spec for path, part in self.named_parts().items()
                for local, spec in part.parameters().items()}

    def checkpoint_specs(self) -> dict[str, ParamSpec]:
        """Checkpoint tensor name -> spec."""
        names = self.config.tensor_names()
        out = {}
        for path, spec in self.parameter_specs().items():
            if path not in names:
                raise ConfigError(f"the configuration gives no checkpoint name for parameter {path}")
            out[names[path]] = spec
        return out

    def new_cache(self, max_tokens: int, max_slots: int | None = None, window_slack: int = 0) -> SequenceCache:
        return SequenceCache(self.cache_needs(), max_tokens=max_tokens, max_slots=max_slots, dtype=self.dtype,
                             device=self.device, window_slack=window_slack)

    # ---- weights
    def load_tensors(self, by_checkpoint_name: dict[str, torch.Tensor]) -> None:
        """Give every part its parameters.  Tensors may live on the CPU or already on the device."""
        names = self.config.tensor_names()
        for path, part in self.named_parts().items():
            local = {}
            for pname in part.parameters():
                local[pname] = by_checkpoint_name[names[f"{path}.{pname}"]]
            part.load(local, self.dtype, self.device)
        self.loaded = True

    def load_folder(self, model_dir: str | Path) -> None:
        expected = {name: spec.shape for name, spec in self.checkpoint_specs().items()}
        tensors = load_checkpoint_tensors(model_dir, expected, self.dtype, set(self.config.optional_tensor_names()))
        self.load_tensors(tensors)

    def load_random(self, seed: int, *, norm_std: float = 0.0, store_dtype: torch.dtype = torch.bfloat16) -> None:
        """Random weights made on the model's device: the same bits as the folder that the random-weights mode
        writes from this seed (``write_random_model(config, seed, dir, norm_std=..., dtype=store_dtype)``)."""
        from ..weights.random_init import random_tensor

        specs = self.checkpoint_specs()
        names = self.config.tensor_names()
        for path, part in self.named_parts().items():
            local = {}
            for pname in part.parameters():
                cname = names[f"{path}.{pname}"]
                local[pname] = random_tensor(cname, specs[cname], seed, self.config.init_std(), norm_std, store_dtype,
                                             self.device)
            part.load(local, self.dtype, self.device)
        self.loaded = True

    # ---- one forward pass over a packed batch
    def forward(self, ctx: StepContext, cache: SequenceCache, logit_rows: torch.Tensor | None) -> torch.Tensor | None:
        """Run the tokens of ``ctx`` through every scheduled block, writing the cache; return float32
        logits [len(logit_rows), vocab] (None when no row is wanted)."""
        if not self.loaded:
            raise WeightError("the model has no weights yet (load_folder / load_random / load_tensors)")
        ws = ctx.workspace
        residual = self.embedding.forward(ctx.tokens, ctx.empty)  # float32 [T, hidden]; lives for the whole pass
        # a block may leave the first norm of the block that runs next to that block's first product
        # (parts/base.py, ScaledRows); blocks that do not offer this are called the plain way
        handed = None
        for k, entry in enumerate(self.schedule):
            view = cache.view(entry.cache) if entry.cache is not None else None
            block = self.blocks[entry.layer]
            mark = ws.mark() if ws is not None else 0
            if block.takes_scaled_rows(ctx):
                nxt = self.blocks[self.schedule[k + 1].layer] if k + 1 < len(self.schedule) else None
                then = nxt.first_norm() if nxt is not None and nxt.takes_scaled_rows(ctx) else None
                handed = block.forward(residual, ctx, view, entry.writes_cache, x_in=handed, then_norm=then)
            else:
                block.forward(residual, ctx, view, entry.writes_cache)
                handed = None
            if ws is not None:
                ws.release(mark)   # the block's intermediate tensors; what it hands on does not come from there
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        x = self.final_norm.forward(residual, ctx.dtype, rows=logit_rows, alloc=ctx.empty)
        return self.head.forward(x)


def parameter_specs_by_checkpoint_name(config: ModelConfig) -> dict[str, ParamSpec]:
    """Checkpoint names and shapes of the model of ``config``; touches no device."""
    from ..config.registry import architecture_of

    arch = architecture_of({"architectures": [config.architecture]})
    model = arch.model_factory(config, torch.bfloat16, "cpu")
    return model.checkpoint_specs()
