"""Registries: architecture name -> (configuration class, model description), and
part name -> part class for every kind of part a layer is put together from.

The reference hard-wires one model (gpu_decoder.cu:163-215 builds exactly the
Qwen2 decoder); here a model is looked up by ``config.json``'s
``architectures[0]`` and described as data (``ModelSpec``), and each part of a
layer is created by name, so another mixer, feed-forward, norm, position
encoding or whole architecture is added by registering it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .model_config import ConfigError, read_config_json

PART_KINDS = ("mixer", "feed_forward", "norm", "position", "block")


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_cls: Any                     # has from_dict(dict) and to_dict()
    describe: Callable[[Any], Any]      # config -> ModelSpec


_ARCHITECTURES: Dict[str, ArchitectureEntry] = {}
_PARTS: Dict[str, Dict[str, Any]] = {k: {} for k in PART_KINDS}


def register_architecture(name: str, config_cls, describe) -> None:
    """Make ``architectures[0] == name`` resolve to ``config_cls`` and ``describe``."""
    _ARCHITECTURES[name] = ArchitectureEntry(name, config_cls, describe)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures():
    return sorted(_ARCHITECTURES)


def lookup_architecture(name: str) -> ArchitectureEntry:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; known: {', '.join(known_architectures()) or '(none)'}"
        ) from None


def register_part(kind: str, name: str):
    """Class decorator: ``@register_part("mixer", "gq_attention")``."""
    if kind not in _PARTS:
        raise ValueError(f"unknown part kind {kind!r}; kinds: {PART_KINDS}")

    def deco(cls):
        _PARTS[kind][name] = cls
        cls.part_kind = kind
        cls.part_name = name
        return cls

    return deco


def unregister_part(kind: str, name: str) -> None:
    _PARTS[kind].pop(name, None)


def create_part(kind: str, name: str, **params):
    try:
        cls = _PARTS[kind][name]
    except KeyError:
        raise ConfigError(
            f"unknown {kind} part {name!r}; known: {', '.join(sorted(_PARTS[kind])) or '(none)'}"
        ) from None
    return cls(**params)


def config_from_dict(d: Mapping[str, Any]):
    """Typed configuration chosen by ``architectures[0]``."""
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of strings")
    return lookup_architecture(archs[0]).config_cls.from_dict(d)


def load_config(model_dir: str):
    """Read ``<model_dir>/config.json`` into the typed configuration of its architecture."""
    return config_from_dict(read_config_json(model_dir))


def describe_model(config):
    """``ModelSpec`` of a typed configuration (see ``config.spec``)."""
    return lookup_architecture(config.architecture).describe(config)
