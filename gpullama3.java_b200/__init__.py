"""gpullama3.java_b200: a small Llama 3 inference library for one NVIDIA B200 (sm_100a).

From a model folder (config.json + safetensors) or a configuration and a seed to generated
tokens: typed configuration and architecture registry, weights by tensor name, a decoder put
together from parts, a paged cache with a slot per sequence, one step function, a generation
loop, samplers, hand-written CUDA kernels in bfloat16 and a true float32 path, and trace replay.
"""
from .config import ConfigError, LlamaConfig, load_config, register_architecture
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "LlamaConfig", "load_config", "register_architecture", "WeightError", "write_random_model"]
