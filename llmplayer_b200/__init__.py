"""llmplayer_b200: a small model library with generation, for one B200.

From a model folder (config.json + model.safetensors) to generated tokens:
typed configuration and architecture registry (config), weights by name
(weights), layers composed of parts (parts), a paged cache with slots (cache),
one step function and the generation loop (engine), samplers (sampling) and the
CUDA kernels for sm_100a (csrc, kernels).
"""
from .errors import (
    CacheError, CacheFull, ConfigError, ExtensionMissing, KernelError, LLMPlayerError, RequestError, WeightError,
)
from .config import LlamaConfig, load_config, register_architecture

__version__ = "0.1.0"


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    if name in ("SamplingParams", "SamplerConfig"):
        from . import sampling
        return getattr(sampling, name)
    if name == "write_random_model":
        from .weights import write_random_model
        return write_random_model
    raise AttributeError(name)
