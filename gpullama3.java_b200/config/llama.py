"""Typed configuration of the Llama 3 decoder, read from ``config.json``.

The reference reads the same quantities from GGUF metadata (model/loader/LlamaModelLoader.java:33-47
of the reference project) into ``LlamaConfiguration`` (model/llama/LlamaConfiguration.java:6-39),
with the same defaults: kv heads = heads when absent, rms eps 1e-5, rope base 10000.  Unlike the
reference (model/loader/ModelLoader.java:234-239) the llama3 rope-scaling numbers are read from
the configuration, never fixed in code."""
from __future__ import annotations

from dataclasses import dataclass

from .base import (ConfigError, LayerSpec, ModelConfig, PartSpec, as_float, as_int, require_keys)
from .registry import register_architecture


@dataclass(frozen=True)
class RopeScaling:
    """The llama3 wavelength rule of inference/operation/RoPE.java:16-28 (reference project)."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @classmethod
    def from_dict(cls, d) -> "RopeScaling | None":
        if d is None:
            return None
        if not isinstance(d, dict):
            raise ConfigError(f"rope_scaling must be an object or null, got {d!r}")
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(f"rope_scaling type {kind!r} is not supported (only 'llama3')")
        require_keys(d, ["factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings"],
                     "rope_scaling")
        s = cls("llama3", as_float(d, "factor"), as_float(d, "low_freq_factor"), as_float(d, "high_freq_factor"),
                as_int(d, "original_max_position_embeddings"))
        if s.factor <= 0 or s.high_freq_factor == s.low_freq_factor or s.low_freq_factor <= 0:
            raise ConfigError(f"rope_scaling has unusable factors: {d!r}")
        return s

    def to_dict(self) -> dict:
        return {"rope_type": self.rope_type, "factor": self.factor, "low_freq_factor": self.low_freq_factor,
                "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position_embeddings}


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling | None
    tie_word_embeddings: bool
    stop_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    rope_pairing: str = "half"
    torch_dtype: str = "bfloat16"
    initializer_range: float = 0.02

    architecture = "LlamaForCausalLM"

    # ---- reading
    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        require_keys(d, ["num_hidden_layers", "hidden_size", "num_attention_heads", "intermediate_size", "vocab_size"],
                     "Llama config.json")
        heads = as_int(d, "num_attention_heads")
        hidden = as_int(d, "hidden_size")
        kv_heads = as_int(d, "num_key_value_heads") if d.get("num_key_value_heads") is not None else heads
        if d.get("head_dim") is not None:
            head_dim = as_int(d, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError(f"hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                                  "and no head_dim is given")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"head_dim {head_dim} must be even for rotary pairs")
        for flag in ("attention_bias", "mlp_bias"):
            if d.get(flag):
                raise ConfigError(f"{flag}=true is not supported: the Llama 3 decoder has no biases")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported (Llama 3 uses 'silu')")
        eos = d.get("eos_token_id")
        if eos is None:
            stop = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            stop = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            stop = tuple(eos)
        else:
            raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {eos!r}")
        pairing = d.get("rope_pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ConfigError(f"rope_pairing must be 'half' or 'interleaved', got {pairing!r}")
        eps = as_float(d, "rms_norm_eps") if d.get("rms_norm_eps") is not None else 1e-5
        theta = as_float(d, "rope_theta") if d.get("rope_theta") is not None else 10000.0
        if eps <= 0 or theta <= 0:
            raise ConfigError("rms_norm_eps and rope_theta must be positive")
        max_pos = as_int(d, "max_position_embeddings") if d.get("max_position_embeddings") is not None else 2048
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if dtype not in ("bfloat16", "float32", "float16"):
            raise ConfigError(f"torch_dtype {dtype!r} is not supported")
        return cls(
            num_hidden_layers=as_int(d, "num_hidden_layers"), hidden_size=hidden, num_attention_heads=heads,
            num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=as_int(d, "intermediate_size"),
            vocab_size=as_int(d, "vocab_size"), max_position_embeddings=max_pos, rms_norm_eps=eps, rope_theta=theta,
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)), stop_token_ids=stop,
            bos_token_id=d.get("bos_token_id"), rope_pairing=pairing, torch_dtype=dtype,
            initializer_range=float(d.get("initializer_range", 0.02)))

    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture], "model_type": "llama",
            "num_hidden_layers": self.num_hidden_layers, "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings, "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "tie_word_embeddings": self.tie_word_embeddings, "hidden_act": "silu", "attention_bias": False,
            "mlp_bias": False, "torch_dtype": self.torch_dtype, "rope_pairing": self.rope_pairing,
            "initializer_range": self.initializer_range,
        }
        if self.stop_token_ids:
            d["eos_token_id"] = list(self.stop_token_ids) if len(self.stop_token_ids) > 1 else self.stop_token_ids[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d

    # ---- derived sizes (model/llama/LlamaConfiguration.java:27-39 of the reference project)
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    # ---- the model as data
    def layer_specs(self) -> list[LayerSpec]:
        norm = self.final_norm()
        position = PartSpec("position", "rope", {
            "head_dim": self.head_dim, "theta": self.rope_theta, "pairing": self.rope_pairing,
            "scaling": self.rope_scaling.to_dict() if self.rope_scaling else None})
        mixer = PartSpec("mixer", "attention", {
            "hidden_size": self.hidden_size, "n_heads": self.num_attention_heads,
            "n_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim, "position": position, "window": None})
        ff = PartSpec("feed_forward", "swiglu", {"hidden_size": self.hidden_size,
                                                 "intermediate_size": self.intermediate_size})
        layer = LayerSpec("pre_norm", {"mixer": mixer, "feed_forward": ff, "mixer_norm": norm, "feed_forward_norm": norm})
        return [layer for _ in range(self.num_hidden_layers)]

    def final_norm(self) -> PartSpec:
        return PartSpec("norm", "rmsnorm", {"dim": self.hidden_size, "eps": self.rms_norm_eps})

    def tensor_names(self) -> dict[str, str]:
        names = {"embedding.table": "model.embed_tokens.weight", "final_norm.weight": "model.norm.weight"}
        if not self.tie_word_embeddings:
            names["head.weight"] = "lm_head.weight"
        for i in range(self.num_hidden_layers):
            p, c = f"layers.{i}.", f"model.layers.{i}."
            names[p + "mixer_norm.weight"] = c + "input_layernorm.weight"
            names[p + "feed_forward_norm.weight"] = c + "post_attention_layernorm.weight"
            for w in ("q", "k", "v", "o"):
                names[p + f"mixer.{w}"] = c + f"self_attn.{w}_proj.weight"
            for w in ("gate", "up", "down"):
                names[p + f"feed_forward.{w}"] = c + f"mlp.{w}_proj.weight"
        return names

    def max_sequence_length(self) -> int:
        # the reference caps every run at the configuration's context length
        # (inference/InferenceEngine.java:75-77, model/llama/LlamaConfiguration.java:49-64 of the reference project)
        return self.max_position_embeddings

    def optional_tensor_names(self) -> set[str]:
        return {"lm_head.weight"} if self.tie_word_embeddings else set()

    def init_std(self) -> float:
        return self.initializer_range


register_architecture("LlamaForCausalLM", LlamaConfig)
