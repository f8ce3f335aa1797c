"""One registry from names to the things a model is made of.

* architectures: the name in ``config.json``'s ``architectures[0]`` -> (configuration class,
  function that turns a configuration into a ``ModelSpec``).  This plays the role of the
  reference's ``ComponentFactory`` (factory/factory.py:12-54) one level up: the reference picks
  an implementation per component type, here a configuration picks parts per layer.
* parts: ``mixer``, ``feed_forward``, ``norm``, ``position``, ``block``, ``embedding``, ``head``
  -> class, by the ``kind`` a ``PartSpec`` names.

Registering is open: a test or a user module can add a mixer or a whole architecture
without touching the package.
"""

from __future__ import annotations

from typing import Callable, Dict, Tuple, Type

from .config.model_config import ConfigError, ModelConfig, read_config_json
from .parts.base import ModelSpec, Part, PartSpec

PART_TYPES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")

_parts: Dict[str, Dict[str, Type[Part]]] = {t: {} for t in PART_TYPES}
_architectures: Dict[str, Tuple[Type[ModelConfig], Callable[[ModelConfig], ModelSpec]]] = {}


def register_part(part_type: str, kind: str):
    """Class decorator: ``@register_part("mixer", "gqa_attention")``."""
    if part_type not in _parts:
        raise ValueError(f"unknown part type '{part_type}' (known: {', '.join(PART_TYPES)})")

    def deco(cls):
        _parts[part_type][kind] = cls
        return cls

    return deco


def create_part(part_type: str, spec: PartSpec, name: str = "") -> Part:
    _load_builtin()
    table = _parts.get(part_type)
    if table is None:
        raise ValueError(f"unknown part type '{part_type}' (known: {', '.join(PART_TYPES)})")
    cls = table.get(spec.kind)
    if cls is None:
        raise ValueError(f"no {part_type} registered as '{spec.kind}' (registered: {', '.join(sorted(table)) or 'none'})")
    return cls(name=name, **spec.params)


def registered_parts(part_type: str):
    return sorted(_parts[part_type])


def register_architecture(name: str, config_cls: Type[ModelConfig]):
    """Function decorator: the function maps a configuration object to a ``ModelSpec``."""

    def deco(fn):
        _architectures[name] = (config_cls, fn)
        return fn

    return deco


def registered_architectures():
    return sorted(_architectures)


def _entry(name: str):
    _load_builtin()
    if name not in _architectures:
        raise ConfigError(
            f"architecture '{name}' is not registered (registered: {', '.join(registered_architectures()) or 'none'})")
    return _architectures[name]


def load_config(folder_or_file: str) -> ModelConfig:
    """Reads config.json and returns the typed configuration of the architecture it names."""
    data = read_config_json(folder_or_file)
    archs = data.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs:
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    config_cls, _ = _entry(archs[0])
    return config_cls.from_dict(data)


def config_from_dict(data: dict) -> ModelConfig:
    archs = data.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs:
        raise ConfigError("config: 'architectures' must be a non-empty list of names")
    config_cls, _ = _entry(archs[0])
    return config_cls.from_dict(data)


def build_model_spec(config: ModelConfig) -> ModelSpec:
    _, builder = _entry(config.architecture)
    return builder(config)


_builtin_loaded = False


def _load_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from .parts import attention, block, embedding, mlp, norm, rope  # noqa: F401  register themselves
        from .models import qwen3  # noqa: F401  registers the architecture
