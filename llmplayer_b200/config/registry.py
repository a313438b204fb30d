"""One registry from an architecture's name to its configuration class.

The reference maps the file's architecture string to an enum constant and
throws on an unknown one (model/ModelArchitecture.java:35-57); the engine is
then picked by an if-chain on that enum (api/LLMEngine.java:89-170). Here the
name in ``config.json`` (``architectures[0]``) selects a configuration class,
and that class alone says how the model is laid out.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Type

from ..errors import ConfigError

_ARCHITECTURES: Dict[str, Type["ArchitectureConfig"]] = {}


class ArchitectureConfig:
    """What every architecture's configuration must offer.

    ``from_dict`` reads the architecture's own config.json keys and validates
    them; ``to_dict`` writes them back (so that a random model folder can be
    made from a configuration); ``layout`` turns the sizes into the parts of
    the model (:class:`llmplayer_b200.parts.specs.ModelLayout`).
    """

    architecture: str = ""

    @classmethod
    def from_dict(cls, raw: dict) -> "ArchitectureConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    def layout(self):
        raise NotImplementedError

    def stop_token_ids(self) -> tuple:
        """Token ids that end a sequence, as far as the configuration knows them."""
        return ()

    def max_positions(self) -> int:
        raise NotImplementedError


def register_architecture(name: str, config_cls: Type[ArchitectureConfig], *, replace: bool = False) -> None:
    if not name:
        raise ConfigError("an architecture needs a name")
    if name in _ARCHITECTURES and not replace and _ARCHITECTURES[name] is not config_cls:
        raise ConfigError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = config_cls


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> tuple:
    return tuple(sorted(_ARCHITECTURES))


def config_class_for(name: str) -> Type[ArchitectureConfig]:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"Unknown architecture: {name!r}; known: {', '.join(known_architectures()) or '(none)'}"
        ) from None


def config_from_dict(raw: dict) -> ArchitectureConfig:
    if not isinstance(raw, dict):
        raise ConfigError("config.json must hold a JSON object")
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError('config.json needs "architectures": ["<name>"]')
    return config_class_for(archs[0]).from_dict(raw)


def load_config(model_dir: str) -> ArchitectureConfig:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as fh:
            raw = json.load(fh)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in {model_dir!r}") from None
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from None
    return config_from_dict(raw)
