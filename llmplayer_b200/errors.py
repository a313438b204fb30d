"""Typed errors of the library.

The reference reports faults as unchecked Java exceptions with a message
(``IllegalArgumentException("Unknown architecture: ...")`` in
model/ModelArchitecture.java:35-57, ``IllegalStateException("Required tensor
not found: ...")`` in model/ModelLoader.java:695-701) and, on a GPU fault,
falls back to the CPU for good (inference/InferenceEngine.java:355-365).
Here every fault has a type, and nothing falls back.
"""


class LLMPlayerError(Exception):
    """Base of every error this library raises on purpose."""


class ConfigError(LLMPlayerError, ValueError):
    """config.json is missing a key, holds a bad value or names an unknown architecture."""


class WeightError(LLMPlayerError, ValueError):
    """The tensors of a model folder do not fit the configuration."""


class CacheFull(LLMPlayerError, RuntimeError):
    """No free slot, page or state row is left for the request."""


class CacheError(LLMPlayerError, RuntimeError):
    """A slot was used in a way its state does not allow (freed twice, not held, ...)."""


class KernelError(LLMPlayerError, RuntimeError):
    """A kernel refused its arguments or the device reported a fault."""


class ExtensionMissing(LLMPlayerError, ImportError):
    """The compiled CUDA library is absent and could not be built."""


class RequestError(LLMPlayerError, ValueError):
    """A step or a generation request is malformed (bad token id, too long, ...)."""
